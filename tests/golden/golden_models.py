"""Two tiny llama models with weights from a plain integer generator, so that anyone can rebuild exactly the
folders the golden outputs were made from (no dependence on a library's random stream)."""
import json
import os
import struct

import numpy as np

GA = {"architectures": ["LlamaForCausalLM"], "hidden_size": 64, "num_hidden_layers": 2, "num_attention_heads": 4,
      "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 176, "vocab_size": 256, "rms_norm_eps": 1e-5,
      "rope_theta": 10000.0, "rope_scaling": None, "max_position_embeddings": 128, "tie_word_embeddings": True,
      "hidden_act": "silu", "torch_dtype": "float32"}
GB = {"architectures": ["LlamaForCausalLM"], "hidden_size": 96, "num_hidden_layers": 3, "num_attention_heads": 3,
      "num_key_value_heads": 1, "head_dim": 32, "intermediate_size": 200, "vocab_size": 387, "rms_norm_eps": 1e-6,
      "rope_theta": 500000.0,
      "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                       "original_max_position_embeddings": 64},
      "max_position_embeddings": 256, "tie_word_embeddings": False, "hidden_act": "silu", "torch_dtype": "float32"}
# biases on q, k, v and o, linear position scaling, a head size (12) that is no multiple of 16
GC = {"architectures": ["LlamaForCausalLM"], "hidden_size": 72, "num_hidden_layers": 2, "num_attention_heads": 6,
      "num_key_value_heads": 2, "head_dim": 12, "intermediate_size": 104, "vocab_size": 211, "rms_norm_eps": 2e-5,
      "rope_theta": 10000.0, "rope_scaling": {"rope_type": "linear", "factor": 2.5}, "max_position_embeddings": 256,
      "tie_word_embeddings": False, "attention_bias": True, "hidden_act": "silu", "torch_dtype": "float32"}
MODELS = {"GA": (GA, 11), "GB": (GB, 12), "GC": (GC, 13)}
TOKENS = {"GA": 40, "GB": 100, "GC": 60}


def lcg_uniform(seed: int, n: int) -> np.ndarray:
    """n values in [-1, 1) from x <- 1664525 x + 1013904223 (mod 2^32), the top 24 bits of each."""
    out = np.empty(n, dtype=np.float64)
    x = seed & 0xFFFFFFFF
    for i in range(n):
        x = (1664525 * x + 1013904223) & 0xFFFFFFFF
        out[i] = (x >> 8) / float(1 << 23) - 1.0
    return out


def tensors_for(cfg: dict, seed: int):
    d, L, H = cfg["hidden_size"], cfg["num_hidden_layers"], cfg["num_attention_heads"]
    K, hd, F, V = cfg["num_key_value_heads"], cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"]
    shapes = [("model.embed_tokens.weight", (V, d))]
    for l in range(L):
        p = f"model.layers.{l}."
        shapes += [(p + "input_layernorm.weight", (d,)), (p + "self_attn.q_proj.weight", (H * hd, d)),
                   (p + "self_attn.k_proj.weight", (K * hd, d)), (p + "self_attn.v_proj.weight", (K * hd, d)),
                   (p + "self_attn.o_proj.weight", (d, H * hd)), (p + "post_attention_layernorm.weight", (d,)),
                   (p + "mlp.gate_proj.weight", (F, d)), (p + "mlp.up_proj.weight", (F, d)), (p + "mlp.down_proj.weight", (d, F))]
        if cfg.get("attention_bias"):
            shapes += [(p + "self_attn.q_proj.bias", (H * hd,)), (p + "self_attn.k_proj.bias", (K * hd,)),
                       (p + "self_attn.v_proj.bias", (K * hd,)), (p + "self_attn.o_proj.bias", (d,))]
    shapes.append(("model.norm.weight", (d,)))
    if not cfg["tie_word_embeddings"]:
        shapes.append(("lm_head.weight", (V, d)))
    out = {}
    for i, (name, shape) in enumerate(shapes):
        u = lcg_uniform(seed * 1000 + i, int(np.prod(shape)))
        vals = 0.3 * u if name.endswith(".bias") else (1.0 + 0.1 * u if len(shape) == 1 else 0.12 * u)
        out[name] = vals.astype(np.float32).reshape(shape)
    return out


def token_ids(name: str):
    cfg, seed = MODELS[name]
    u = lcg_uniform(seed + 500, TOKENS[name])
    return [int((v + 1.0) / 2.0 * cfg["vocab_size"]) % cfg["vocab_size"] for v in u]


def build_folder(path: str, name: str) -> str:
    cfg, seed = MODELS[name]
    os.makedirs(path, exist_ok=True)
    tensors = tensors_for(cfg, seed)
    header, off = {}, 0
    for n, a in tensors.items():
        header[n] = {"dtype": "F32", "shape": list(a.shape), "data_offsets": [off, off + a.nbytes]}
        off += a.nbytes
    blob = json.dumps(header).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(os.path.join(path, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(blob)) + blob)
        for a in tensors.values():
            f.write(a.astype("<f4").tobytes())
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    return path
