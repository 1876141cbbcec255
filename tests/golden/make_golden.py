#!/usr/bin/env python3
"""Makes tests/golden/*.npz: logits of the REFERENCE's own CPU model code on three tiny llama models.

How it was run (offline, CPU only).  The reference's sources were copied to a scratch folder and a small
driver was compiled against them, with the CPU-only backend stub in place of the CUDA backend (the source
list is the reference Makefile's CPU_STUB_SRC, Makefile:808-812, without src/main.c and the server files):

    gcc -O2 -fno-fast-math -std=gnu11 -I src src/gguf.c src/compat.c src/quants.c src/instances.c \\
        src/tokenizer.c src/model.c src/sample.c src/vramreg.c src/template.c src/jsonmode.c src/schema.c \\
        src/quantize.c src/engine.c src/json.c src/envelope.c src/gpu_none.c driver.c -o driver -lm -lpthread -ldl

driver.c (DRIVER_C below) loads a GGUF with `model_load` (GPU off) and calls `model_forward(m, tok[t], t)` for
t = 0..n-1, writing every position's logits -- the same calls as tests/test_gpu_identity.c:81-105.

    python tests/golden/make_golden.py --driver /path/to/driver

This script writes each model as GGUF v3 the way the reference expects a llama model: metadata keys as in
scripts/make-test-model.py:344-363 plus `attention.key_length`; tensors F32 with ne = [in, out], data aligned
to 32 bytes (:533-555); attn_q / attn_k rows permuted per head for the adjacent-pair rotation that arch
"llama" uses (src/model.c:1464-1466: new row 2j <- old row j, new row 2j+1 <- old row j + hd/2, which leaves
every score unchanged); `rope_freqs.weight` = the llama3 divisors (src/model.c:291-297); no `output.weight`
when the head is tied (src/model.c:2353-2354).

The reference rounds K and V to float16 in its cache even on the CPU (src/model.c:6306-6309), so its logits
agree with a float32 implementation to about 1e-3 of their range, not tighter; the bound used by the test is
the reference's own, mean |diff| / range <= 2e-3 (tests/test_gpu_identity.c:60).
"""
import argparse
import os
import struct
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))
import golden_models as gm  # noqa: E402
from plain_llama import rope_inv_freq  # noqa: E402

DRIVER_C = r'''
#include "model.h"
#include "fp16.h"
#include "gpu.h"
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
int main(int argc, char **argv) {
    if (argc < 4) return 2;
    FILE *f = fopen(argv[2], "rb"); if (!f) return 2;
    fseek(f, 0, SEEK_END); long nb = ftell(f); fseek(f, 0, SEEK_SET);
    int n = (int)(nb / 4); int32_t *tok = malloc(nb); if (fread(tok, 4, n, f) != (size_t)n) return 2; fclose(f);
    f16_init();
    model_t m; memset(&m, 0, sizeof(m));
    model_params p; memset(&p, 0, sizeof(p));
    p.gpu_mode = GPU_OFF; p.n_ctx = n + 8; p.n_batch = 1;
    if (!model_load(&m, argv[1], &p)) return 1;
    FILE *o = fopen(argv[3], "wb");
    for (int t = 0; t < n; t++) {
        float *lg = model_forward(&m, tok[t], t);
        if (!lg) return 1;
        fwrite(lg, sizeof(float), m.n_vocab, o);
    }
    fclose(o); model_free(&m); return 0;
}
'''


def s(x: str) -> bytes:
    b = x.encode()
    return struct.pack("<Q", len(b)) + b


def kv_u32(k, v): return s(k) + struct.pack("<II", 4, v)
def kv_f32(k, v): return s(k) + struct.pack("<If", 6, v)
def kv_str(k, v): return s(k) + struct.pack("<I", 8) + s(v)


def permute_rows(w: np.ndarray, heads: int, hd: int) -> np.ndarray:
    out = np.empty_like(w)
    half = hd // 2
    for h in range(heads):
        for j in range(half):
            out[h * hd + 2 * j] = w[h * hd + j]
            out[h * hd + 2 * j + 1] = w[h * hd + j + half]
    return out


def write_gguf(path: str, cfg: dict, tensors: dict) -> None:
    d, L, H = cfg["hidden_size"], cfg["num_hidden_layers"], cfg["num_attention_heads"]
    K, hd = cfg["num_key_value_heads"], cfg["head_dim"]
    a = "llama"
    kvs = [kv_str("general.architecture", a), kv_u32(f"{a}.block_count", L), kv_u32(f"{a}.context_length", cfg["max_position_embeddings"]),
           kv_u32(f"{a}.embedding_length", d), kv_u32(f"{a}.feed_forward_length", cfg["intermediate_size"]),
           kv_u32(f"{a}.attention.head_count", H), kv_u32(f"{a}.attention.head_count_kv", K),
           kv_u32(f"{a}.attention.key_length", hd), kv_u32(f"{a}.attention.value_length", hd),
           kv_f32(f"{a}.attention.layer_norm_rms_epsilon", cfg["rms_norm_eps"]), kv_f32(f"{a}.rope.freq_base", cfg["rope_theta"])]
    sc = cfg.get("rope_scaling") or {}
    if sc.get("rope_type", sc.get("type")) == "linear":            # src/model.c:317-326, 361-362
        kvs += [kv_str(f"{a}.rope.scaling.type", "linear"), kv_f32(f"{a}.rope.scaling.factor", sc["factor"])]
    out = [("token_embd.weight", tensors["model.embed_tokens.weight"]), ("output_norm.weight", tensors["model.norm.weight"])]
    if "lm_head.weight" in tensors:
        out.append(("output.weight", tensors["lm_head.weight"]))
    if sc.get("rope_type", sc.get("type")) == "llama3":
        plain = rope_inv_freq(cfg["rope_theta"], hd)
        scaled = rope_inv_freq(cfg["rope_theta"], hd, cfg["rope_scaling"])
        out.append(("rope_freqs.weight", (plain.astype(np.float64) / scaled.astype(np.float64)).astype(np.float32)))
    for l in range(L):
        p = f"model.layers.{l}."
        out += [(f"blk.{l}.attn_norm.weight", tensors[p + "input_layernorm.weight"]),
                (f"blk.{l}.attn_q.weight", permute_rows(tensors[p + "self_attn.q_proj.weight"], H, hd)),
                (f"blk.{l}.attn_k.weight", permute_rows(tensors[p + "self_attn.k_proj.weight"], K, hd)),
                (f"blk.{l}.attn_v.weight", tensors[p + "self_attn.v_proj.weight"]),
                (f"blk.{l}.attn_output.weight", tensors[p + "self_attn.o_proj.weight"]),
                (f"blk.{l}.ffn_norm.weight", tensors[p + "post_attention_layernorm.weight"]),
                (f"blk.{l}.ffn_gate.weight", tensors[p + "mlp.gate_proj.weight"]),
                (f"blk.{l}.ffn_up.weight", tensors[p + "mlp.up_proj.weight"]),
                (f"blk.{l}.ffn_down.weight", tensors[p + "mlp.down_proj.weight"])]
        if cfg.get("attention_bias"):
            # optional tensors (src/model.c:2832-2837); the q and k biases follow their rows' permutation
            out += [(f"blk.{l}.attn_q.bias", permute_rows(tensors[p + "self_attn.q_proj.bias"].reshape(-1, 1), H, hd).reshape(-1)),
                    (f"blk.{l}.attn_k.bias", permute_rows(tensors[p + "self_attn.k_proj.bias"].reshape(-1, 1), K, hd).reshape(-1)),
                    (f"blk.{l}.attn_v.bias", tensors[p + "self_attn.v_proj.bias"]),
                    (f"blk.{l}.attn_output.bias", tensors[p + "self_attn.o_proj.bias"])]
    header = struct.pack("<IIQQ", 0x46554747, 3, len(out), len(kvs))
    info, off = b"", 0
    for name, arr in out:
        ne = list(reversed(arr.shape))              # ne[0] is the contiguous (input) axis
        info += s(name) + struct.pack("<I", len(ne)) + b"".join(struct.pack("<Q", x) for x in ne) + struct.pack("<IQ", 0, off)
        off = (off + arr.nbytes + 31) & ~31
    head = header + b"".join(kvs) + info
    with open(path, "wb") as f:
        f.write(head + b"\0" * ((-len(head)) % 32))
        for _, arr in out:
            raw = arr.astype("<f4").tobytes()
            f.write(raw + b"\0" * ((-len(raw)) % 32))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--driver", required=True, help="the compiled driver (see this file's header)")
    args = ap.parse_args()
    for name, (cfg, seed) in gm.MODELS.items():
        with tempfile.TemporaryDirectory() as d:
            tensors = gm.tensors_for(cfg, seed)
            gguf = os.path.join(d, "m.gguf")
            write_gguf(gguf, cfg, tensors)
            toks = np.array(gm.token_ids(name), dtype="<i4")
            toks.tofile(os.path.join(d, "tok.i32"))
            subprocess.run([args.driver, gguf, os.path.join(d, "tok.i32"), os.path.join(d, "out.f32")], check=True)
            logits = np.fromfile(os.path.join(d, "out.f32"), dtype="<f4").reshape(len(toks), cfg["vocab_size"])
        # keep the file small: every fourth position, float16 storage of float32 values would lose digits, so float32
        keep = np.arange(3, len(toks), 4)
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), tokens=toks, positions=keep, logits=logits[keep])
        print(name, logits.shape, "kept", len(keep), "range", float(logits.max() - logits.min()))


if __name__ == "__main__":
    main()
