"""Tiny configurations of the architecture for the tests, and folders of random weights for them.

A, B and C differ in every size and option: layers, width, heads and groups, head size, inner width
(no power of two), vocabulary, theta and its scaling, the norms' eps, tied or untied head, biases,
and (C) a window on some layers.
"""
import copy
import os

import torch

from xyntetik_runner_b200.architectures.llama import build_llama
from xyntetik_runner_b200.config.llama import LlamaConfig
from xyntetik_runner_b200.weights.loader import write_model_folder

TINY_A = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 64, "num_hidden_layers": 2, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 176, "vocab_size": 256, "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0, "rope_scaling": None, "max_position_embeddings": 1024, "tie_word_embeddings": True,
    "hidden_act": "silu", "torch_dtype": "float32", "bos_token_id": 1, "eos_token_id": 2,
}
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 96, "num_hidden_layers": 3, "num_attention_heads": 3,
    "num_key_value_heads": 1, "head_dim": 32, "intermediate_size": 200, "vocab_size": 387, "rms_norm_eps": 1e-6,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
    "max_position_embeddings": 1024, "tie_word_embeddings": False, "hidden_act": "silu", "torch_dtype": "float32",
    "eos_token_id": [5, 7],
}
# six heads in two groups, head size 48 (a multiple of 16 that is no power of two), biases, and a window
# of 24 keys on layers 0 and 2 (two cache groups)
TINY_C = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 80, "num_hidden_layers": 3, "num_attention_heads": 6,
    "num_key_value_heads": 2, "head_dim": 48, "intermediate_size": 136, "vocab_size": 301, "rms_norm_eps": 3e-6,
    "rope_theta": 25000.0, "rope_scaling": None, "max_position_embeddings": 1024, "tie_word_embeddings": False,
    "attention_bias": True, "hidden_act": "silu", "torch_dtype": "float32", "sliding_window": 24,
    "layer_types": ["sliding_attention", "full_attention", "sliding_attention"],
}
# head sizes that are no multiple of 16 (config.json allows any even size, src/model.c:2316-2322): 24 with as many
# kv heads as heads, and 100 -- the head size of a 3,200-wide model with 32 heads -- with biases and linear
# position scaling
TINY_D = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 72, "num_hidden_layers": 2, "num_attention_heads": 3,
    "num_key_value_heads": 3, "head_dim": 24, "intermediate_size": 104, "vocab_size": 211, "rms_norm_eps": 2e-5,
    "rope_theta": 10000.0, "rope_scaling": None, "max_position_embeddings": 1024, "tie_word_embeddings": True,
    "hidden_act": "silu", "torch_dtype": "float32",
}
TINY_E = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 200, "num_hidden_layers": 2, "num_attention_heads": 2,
    "num_key_value_heads": 1, "head_dim": 100, "intermediate_size": 144, "vocab_size": 150, "rms_norm_eps": 1e-6,
    "rope_theta": 30000.0, "rope_scaling": {"rope_type": "linear", "factor": 2.5}, "max_position_embeddings": 1024,
    "tie_word_embeddings": False, "attention_bias": True, "hidden_act": "silu", "torch_dtype": "float32",
}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E}
SEEDS = {"A": 0, "B": 1, "C": 2, "D": 3, "E": 4}


def make_folder(path: str, name: str, dtype: str = "float32", std: float = 0.1) -> str:
    """Write config.json + model.safetensors for tiny configuration `name` with weights of `dtype`."""
    d = copy.deepcopy(CONFIGS[name])
    d["torch_dtype"] = dtype
    cfg = LlamaConfig.from_dict(d)
    specs = build_llama(cfg).tensor_specs()
    # biases are drawn too (zeros would hide them)
    specs = {n: (s if s.init != "zeros" else type(s)(s.shape, s.kind, "normal")) for n, s in specs.items()}
    tdt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    write_model_folder(path, cfg.to_dict(), specs, SEEDS[name], tdt, std=std, norm_jitter=0.1)
    return path
