"""The reference arm of bench.py: the UNMODIFIED reference program on the benchmark's model shape.

The reference (Joakimpalm-Zen/xyntetik-runner) is a C program that reads GGUF files and brings its own CUDA
backend (driver API through dlopen, kernels as PTX inside the binary, src/cuda.c:40-41, src/kernels_ptx.h), so it
builds with the C compiler alone:

    cp -r <reference> /tmp/xr_ref && make -C /tmp/xr_ref runner CC=gcc ARCH_FLAGS=-march=x86-64-v3
    cp /tmp/xr_ref/runner baseline/_ref/runner

This module writes a GGUF v3 file of the benchmark shape with random bfloat16 weights (metadata keys as the
reference's fixture generator writes them, scripts/make-test-model.py:344-363; a byte-level vocabulary, so that its
own filler prompt tokenises to well over 512 tokens) and runs the reference's stock benchmark mode

    runner -m FILE --bench-json -n N -c CONTEXT

(src/main.c:1435-1515): a 512-token prompt through its chunked prefill, then N tokens decoded one by one, one
sequence -- its command line has no batch of sequences.  Nothing of this repository's engine is on that path; torch
is used to draw the weights only.  Q and K rows are not permuted for the reference's adjacent-pair rotation: with
random weights the permuted matrix has the same law, and speed does not depend on it.
"""
from __future__ import annotations

import json
import os
import shutil
import struct
import subprocess
import tempfile
import time
from typing import Dict, Iterable, List, Optional, Tuple

HERE = os.path.dirname(os.path.abspath(__file__))
RUNNER = os.path.join(HERE, "_ref", "runner")
REFERENCE_SOURCE = os.environ.get("XYNTETIK_REFERENCE_SRC", "")      # the reference's source tree, to build the binary from when it is missing
GGUF_F32, GGUF_BF16 = 0, 30            # tensor type codes (src/quants.h:22)


def ensure_runner() -> Tuple[Optional[str], str]:
    """(path of the reference binary, how it was had) or (None, why not)."""
    if os.path.isfile(RUNNER) and os.access(RUNNER, os.X_OK):
        return RUNNER, "built beforehand (baseline/_ref/runner)"
    if not REFERENCE_SOURCE or not os.path.isdir(os.path.join(REFERENCE_SOURCE, "src")):
        return None, "baseline/_ref/runner is not there and XYNTETIK_REFERENCE_SRC does not name the reference's source tree"
    if shutil.which("make") is None or shutil.which("gcc") is None:
        return None, "make or gcc is not installed"
    work = tempfile.mkdtemp(prefix="xr_ref_build_")
    try:
        src = os.path.join(work, "ref")
        shutil.copytree(REFERENCE_SOURCE, src, symlinks=True)
        r = subprocess.run(["make", "-C", src, "runner", "CC=gcc", "ARCH_FLAGS=-march=x86-64-v3"], capture_output=True, text=True)
        if r.returncode != 0 or not os.path.isfile(os.path.join(src, "runner")):
            return None, "building the reference failed: " + (r.stderr.strip().splitlines() or ["(no message)"])[-1][:200]
        os.makedirs(os.path.dirname(RUNNER), exist_ok=True)
        shutil.copy2(os.path.join(src, "runner"), RUNNER)
        return RUNNER, "built now from the reference's sources"
    finally:
        shutil.rmtree(work, ignore_errors=True)


# ---- GGUF v3 ---------------------------------------------------------------------------------------------
def _s(x: str) -> bytes:
    b = x.encode()
    return struct.pack("<Q", len(b)) + b


def _kv_u32(k, v): return _s(k) + struct.pack("<II", 4, v)
def _kv_f32(k, v): return _s(k) + struct.pack("<If", 6, v)
def _kv_str(k, v): return _s(k) + struct.pack("<I", 8) + _s(v)
def _kv_bool(k, v): return _s(k) + struct.pack("<IB", 7, 1 if v else 0)


def _kv_arr_str(k, items):
    return _s(k) + struct.pack("<IIQ", 9, 8, len(items)) + b"".join(_s(it) for it in items)


def _kv_arr(k, code, fmt, items):
    return _s(k) + struct.pack("<IIQ", 9, code, len(items)) + struct.pack(f"<{len(items)}{fmt}", *items)


def tensor_list(cfg: dict) -> List[Tuple[str, Tuple[int, ...], int]]:
    """(reference tensor name, shape [out, in] or [n], type code) in file order (names: src/model.c:2332-2353, 2422-2427)."""
    d, L, H = cfg["hidden_size"], cfg["num_hidden_layers"], cfg["num_attention_heads"]
    K, hd, F, V = cfg["num_key_value_heads"], cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"]
    out = [("token_embd.weight", (V, d), GGUF_BF16), ("output_norm.weight", (d,), GGUF_F32)]
    if not cfg.get("tie_word_embeddings"):
        out.append(("output.weight", (V, d), GGUF_BF16))
    for l in range(L):
        out += [(f"blk.{l}.attn_norm.weight", (d,), GGUF_F32), (f"blk.{l}.attn_q.weight", (H * hd, d), GGUF_BF16),
                (f"blk.{l}.attn_k.weight", (K * hd, d), GGUF_BF16), (f"blk.{l}.attn_v.weight", (K * hd, d), GGUF_BF16),
                (f"blk.{l}.attn_output.weight", (d, H * hd), GGUF_BF16), (f"blk.{l}.ffn_norm.weight", (d,), GGUF_F32),
                (f"blk.{l}.ffn_gate.weight", (F, d), GGUF_BF16), (f"blk.{l}.ffn_up.weight", (F, d), GGUF_BF16),
                (f"blk.{l}.ffn_down.weight", (d, F), GGUF_BF16)]
    return out


def write_gguf(path: str, cfg: dict, seed: int, std: float = 0.02, device: str = "cuda:0") -> int:
    """Write the model as GGUF v3 with arch "llama"; matrices ~ N(0, std) in bfloat16, norm weights 1 in float32.
    Returns the file's size in bytes."""
    import torch
    a, V = "llama", cfg["vocab_size"]
    vocab = ["<unk>", "<s>", "</s>"] + [f"<0x{i:02X}>" for i in range(256)]
    types = [2, 3, 3] + [6] * 256                      # unknown, control, control, bytes (src/tokenizer.c:11-12)
    vocab += [f"<unused_{i}>" for i in range(len(vocab), V)]
    types += [5] * (V - len(types))
    kvs = [_kv_str("general.architecture", a), _kv_u32(f"{a}.block_count", cfg["num_hidden_layers"]),
           _kv_u32(f"{a}.context_length", cfg["max_position_embeddings"]), _kv_u32(f"{a}.embedding_length", cfg["hidden_size"]),
           _kv_u32(f"{a}.feed_forward_length", cfg["intermediate_size"]), _kv_u32(f"{a}.attention.head_count", cfg["num_attention_heads"]),
           _kv_u32(f"{a}.attention.head_count_kv", cfg["num_key_value_heads"]), _kv_u32(f"{a}.attention.key_length", cfg["head_dim"]),
           _kv_u32(f"{a}.attention.value_length", cfg["head_dim"]),
           _kv_f32(f"{a}.attention.layer_norm_rms_epsilon", cfg["rms_norm_eps"]), _kv_f32(f"{a}.rope.freq_base", cfg["rope_theta"]),
           _kv_str("tokenizer.ggml.model", "llama"), _kv_arr_str("tokenizer.ggml.tokens", vocab[:V]),
           _kv_arr("tokenizer.ggml.scores", 6, "f", [0.0] * V), _kv_arr("tokenizer.ggml.token_type", 5, "i", types[:V]),
           _kv_u32("tokenizer.ggml.bos_token_id", 1), _kv_u32("tokenizer.ggml.eos_token_id", 2),
           _kv_bool("tokenizer.ggml.add_bos_token", True)]
    tensors = tensor_list(cfg)
    info, off = b"", 0
    for name, shape, code in tensors:
        ne = list(reversed(shape))                      # ne[0] is the contiguous (input) axis
        n = 1
        for x in shape:
            n *= x
        info += _s(name) + struct.pack("<I", len(ne)) + b"".join(struct.pack("<Q", x) for x in ne) + struct.pack("<IQ", code, off)
        off = (off + n * (4 if code == GGUF_F32 else 2) + 31) & ~31
    head = struct.pack("<IIQQ", 0x46554747, 3, len(tensors), len(kvs)) + b"".join(kvs) + info
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    with open(path, "wb") as f:
        f.write(head + b"\0" * ((-len(head)) % 32))
        for name, shape, code in tensors:
            if code == GGUF_F32:
                raw = torch.ones(shape, dtype=torch.float32).numpy().tobytes()
                f.write(raw + b"\0" * ((-len(raw)) % 32))
                continue
            rows = max(1, (1 << 27) // shape[1])       # pieces of at most 128 Mi elements
            written = 0
            for r0 in range(0, shape[0], rows):
                r1 = min(shape[0], r0 + rows)
                t = torch.empty((r1 - r0, shape[1]), dtype=torch.float32, device=device).normal_(0.0, std, generator=gen)
                raw = t.to(torch.bfloat16).cpu().view(torch.int16).numpy()
                f.write(memoryview(raw))
                written += raw.nbytes
            f.write(b"\0" * ((-written) % 32))
        return f.tell()


def scratch_dir(need_bytes: int) -> Optional[str]:
    """A folder with room for the model file: memory-backed if there is room, else the temporary folder."""
    for d in ("/dev/shm", tempfile.gettempdir()):
        try:
            if os.path.isdir(d) and shutil.disk_usage(d).free > need_bytes * 1.05:
                return d
        except OSError:
            pass
    return None


def run(cfg: dict, seed: int, n_predict: int, context: int, timeout_s: int = 900, device: str = "cuda:0") -> Dict[str, object]:
    """Write the model, run the reference's --bench-json on it, and return its own JSON (plus `how`, `file_gb`,
    `write_s`, `run_s`), or {"unavailable": why}."""
    runner, how = ensure_runner()
    if runner is None:
        return {"unavailable": how}
    d, L, H, K = cfg["hidden_size"], cfg["num_hidden_layers"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    params = cfg["vocab_size"] * d * (1 if cfg.get("tie_word_embeddings") else 2) + \
        L * (d * (H + 2 * K) * cfg["head_dim"] + H * cfg["head_dim"] * d + 3 * d * cfg["intermediate_size"])
    where = scratch_dir(2 * params + (64 << 20))
    if where is None:
        return {"unavailable": f"no folder with {2 * params / 1e9:.1f} GB free for the reference's model file"}
    path = os.path.join(where, f"xr_ref_bench_{os.getpid()}.gguf")
    try:
        t0 = time.perf_counter()
        size = write_gguf(path, cfg, seed, device=device)
        write_s = time.perf_counter() - t0
        import torch
        torch.cuda.empty_cache()
        cmd = [runner, "-m", path, "--bench-json", "-n", str(n_predict), "-c", str(context), "--gpu", "auto"]
        t0 = time.perf_counter()
        try:
            r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout_s)
        except subprocess.TimeoutExpired:
            return {"unavailable": f"the reference did not finish within {timeout_s} s", "cmd": " ".join(cmd[:1] + cmd[3:])}
        run_s = time.perf_counter() - t0
        line = next((ln for ln in reversed(r.stdout.strip().splitlines()) if ln.startswith("{")), None)
        if r.returncode != 0 or line is None:
            msg = (r.stderr.strip().splitlines() or r.stdout.strip().splitlines() or ["(no output)"])[-1][:300]
            return {"unavailable": f"the reference exited with {r.returncode}: {msg}"}
        out = json.loads(line)
        out.update({"how": how, "file_gb": size / 1e9, "write_s": write_s, "run_s": run_s,
                    "stderr_tail": r.stderr.strip().splitlines()[-3:]})
        return out
    finally:
        try:
            os.remove(path)
        except OSError:
            pass
