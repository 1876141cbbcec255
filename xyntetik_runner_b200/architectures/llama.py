"""The dense Llama decoder as a list of parts chosen from its configuration.

What is fixed here is what the reference fixes for llama in code: pre-norm
placement with two residual additions (src/model.c:6350-6352, 6421-6423), a
SiLU gate (`ACT_SILU`, src/model.h:20), scale 1/sqrt(head_dim)
(src/model.h:464-467), causal attention with kv head = head / (H/K)
(src/model.c:3553), no embedding scale and no logit cap (src/model.c:1467-1469).
Every number comes from the configuration.  Tensor names are those of a
config.json + safetensors checkpoint of this architecture.
"""
from __future__ import annotations

from ..config.llama import LlamaConfig
from ..config.registry import register_architecture
from ..engine.model import ModelPlan, ScheduleEntry
from ..parts import Embedding, GQAAttention, Head, PreNormBlock, RMSNorm, Rope, SwiGLU


def build_llama(cfg: LlamaConfig) -> ModelPlan:
    embedding = Embedding(cfg.vocab_size, cfg.hidden_size, "model.embed_tokens.weight")
    blocks = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        rope = Rope(cfg.head_dim, cfg.rope_theta, scaling=cfg.rope_scaling)
        mixer = GQAAttention(cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                             position=rope, prefix=p + "self_attn.", bias=cfg.attention_bias,
                             window=cfg.layer_window(i))
        ffn = SwiGLU(cfg.hidden_size, cfg.intermediate_size, prefix=p + "mlp.")
        blocks.append(PreNormBlock(RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, p + "input_layernorm.weight"), mixer,
                                   RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, p + "post_attention_layernorm.weight"), ffn))
    final_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, "model.norm.weight")
    if cfg.tie_word_embeddings:
        head = Head(cfg.vocab_size, cfg.hidden_size, tied_to=embedding)
    else:
        head = Head(cfg.vocab_size, cfg.hidden_size, name="lm_head.weight")
    return ModelPlan(embedding=embedding, blocks=blocks,
                     schedule=[ScheduleEntry(layer=i) for i in range(cfg.num_hidden_layers)],
                     final_norm=final_norm, head=head, width=cfg.hidden_size, vocab_size=cfg.vocab_size,
                     max_positions=cfg.max_position_embeddings, stop_ids=tuple(cfg.eos_token_ids),
                     bos_id=cfg.bos_token_id)


def override_llama(cfg: LlamaConfig, rope_base=None, rope_scale=None) -> LlamaConfig:
    """The reference's run-time overrides: another frequency base (--rope-base, src/model.c:282) and linear position
    scaling by a factor in place of the configuration's scaling (--rope-scale, src/model.c:324-326)."""
    import dataclasses
    from ..config.llama import RopeScaling
    if rope_base is not None:
        cfg = dataclasses.replace(cfg, rope_theta=float(rope_base))
    if rope_scale is not None:
        cfg = dataclasses.replace(cfg, rope_scaling=RopeScaling(rope_type="linear", factor=float(rope_scale)))
    return cfg


register_architecture("LlamaForCausalLM", LlamaConfig.from_dict, build_llama, override=override_llama, replace=True)
