"""Typed configuration of the dense Llama decoder, read from config.json.

Every size and constant the model uses is a field here; nothing in the parts or
kernels carries a Llama number of its own.  The admission rules follow the
reference's geometry gate (src/model.c:2295-2329: every dimension present and
bounded by 2^20, ``n_head % n_head_kv == 0``, ``n_head_kv <= n_head``) and its
hyper-parameter defaults (src/model.c:1422-1470: kv heads default to heads,
head size to width / heads, eps 1e-5, theta 10000).
"""
from __future__ import annotations

import json
import os
from .base import ConfigError, read_config_json  # noqa: F401  (both are also importable from here)
from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple

DIM_MAX = 1 << 20          # per-axis ceiling, src/model.c:31
LAYERS_MAX = 100000        # src/model.c:1429-1433


@dataclass(frozen=True)
class RopeScaling:
    """``rope_scaling``.  Type ``llama3``: per-frequency divisors.  The reference consumes these as a
    ``rope_freqs.weight`` tensor written by the converter (src/model.c:291-297); here they are computed
    from the four numbers below when the position table is built.  Type ``linear``: every frequency is
    divided by ``factor`` (src/model.c:361-362); the other three numbers are unused.
    """
    rope_type: str
    factor: float
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 0


@dataclass(frozen=True)
class LlamaConfig:
    architecture: str
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Optional[RopeScaling]
    max_position_embeddings: int
    tie_word_embeddings: bool
    attention_bias: bool
    hidden_act: str
    torch_dtype: str
    bos_token_id: Optional[int]
    eos_token_ids: Tuple[int, ...]
    # None = every layer attends to all earlier keys.  With a window, the
    # layers named "sliding_attention" in layer_types see the last
    # `sliding_window` keys only (the reference keeps a per-layer flag for
    # this, src/model.h:229-235).
    sliding_window: Optional[int] = None
    layer_types: Optional[Tuple[str, ...]] = None
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)

    # ---- derived sizes -------------------------------------------------
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def layer_window(self, layer: int) -> Optional[int]:
        """Window of one layer, or None when it attends to everything."""
        if self.sliding_window is None:
            return None
        if self.layer_types is None:
            return self.sliding_window
        return self.sliding_window if self.layer_types[layer] == "sliding_attention" else None

    # ---- reading ---------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "LlamaConfig":
        def need(key: str, kind):
            if key not in d or d[key] is None:
                raise ConfigError(f"config.json: missing key '{key}'")
            return _typed(key, d[key], kind)

        def opt(key: str, kind, default):
            if key not in d or d[key] is None:
                return default
            return _typed(key, d[key], kind)

        archs = d.get("architectures")
        if not isinstance(archs, list) or len(archs) != 1 or not isinstance(archs[0], str):
            raise ConfigError("config.json: 'architectures' must be a list holding one name")
        hidden = need("hidden_size", int)
        layers = need("num_hidden_layers", int)
        heads = need("num_attention_heads", int)
        if heads < 1:
            raise ConfigError("config.json: num_attention_heads must be >= 1")
        kv_heads = opt("num_key_value_heads", int, heads)
        head_dim = opt("head_dim", int, hidden // heads)
        inter = need("intermediate_size", int)
        vocab = need("vocab_size", int)
        eps = need("rms_norm_eps", float)
        theta = opt("rope_theta", float, 10000.0)
        max_pos = need("max_position_embeddings", int)
        tie = opt("tie_word_embeddings", bool, False)
        attn_bias = opt("attention_bias", bool, False)
        if opt("mlp_bias", bool, False):
            raise ConfigError("config.json: mlp_bias=true is not supported "
                              "(the reference passes no feed-forward bias, src/model.c:6399-6407)")
        act = opt("hidden_act", str, "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act '{act}' is not supported (only 'silu')")
        dtype = opt("torch_dtype", str, opt("dtype", str, "bfloat16"))
        if dtype not in ("bfloat16", "float32", "float16"):
            raise ConfigError(f"config.json: torch_dtype '{dtype}' is not supported")

        scaling = None
        rs = d.get("rope_scaling")
        if rs is not None:
            if not isinstance(rs, Mapping):
                raise ConfigError("config.json: rope_scaling must be an object or null")
            kind = rs.get("rope_type", rs.get("type"))
            if kind == "default":
                rs = None                     # "default" names the unscaled table
            elif kind == "linear":
                try:
                    scaling = RopeScaling(rope_type="linear", factor=float(rs["factor"]))
                except KeyError as e:
                    raise ConfigError(f"config.json: rope_scaling lacks {e}") from None
                if not scaling.factor > 0:
                    raise ConfigError("config.json: rope_scaling factor must be positive")
                rs = None
            elif kind != "llama3":
                raise ConfigError(f"config.json: rope_scaling type '{kind}' is not supported (only 'llama3' and 'linear')")
        if rs is not None:
            try:
                scaling = RopeScaling(
                    rope_type="llama3",
                    factor=float(rs["factor"]),
                    low_freq_factor=float(rs["low_freq_factor"]),
                    high_freq_factor=float(rs["high_freq_factor"]),
                    original_max_position_embeddings=int(rs["original_max_position_embeddings"]),
                )
            except KeyError as e:
                raise ConfigError(f"config.json: rope_scaling lacks {e}") from None
            if (scaling.factor <= 0 or scaling.original_max_position_embeddings < 1
                    or scaling.high_freq_factor <= scaling.low_freq_factor
                    or scaling.low_freq_factor <= 0):
                raise ConfigError("config.json: rope_scaling values out of range "
                                  "(need factor > 0, 0 < low_freq_factor < high_freq_factor)")

        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, list) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError("config.json: eos_token_id must be an integer or a list of integers")
        bos = opt("bos_token_id", int, None)

        window = opt("sliding_window", int, None)
        ltypes = d.get("layer_types")
        if ltypes is not None:
            if (not isinstance(ltypes, list) or
                    any(t not in ("full_attention", "sliding_attention") for t in ltypes)):
                raise ConfigError("config.json: layer_types must list 'full_attention' / 'sliding_attention'")
            ltypes = tuple(ltypes)

        known = {
            "architectures", "hidden_size", "num_hidden_layers", "num_attention_heads",
            "num_key_value_heads", "head_dim", "intermediate_size", "vocab_size", "rms_norm_eps",
            "rope_theta", "rope_scaling", "max_position_embeddings", "tie_word_embeddings",
            "attention_bias", "mlp_bias", "hidden_act", "torch_dtype", "dtype", "bos_token_id",
            "eos_token_id", "sliding_window", "layer_types",
        }
        cfg = cls(
            architecture=archs[0], hidden_size=hidden, num_hidden_layers=layers,
            num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim,
            intermediate_size=inter, vocab_size=vocab, rms_norm_eps=eps, rope_theta=theta,
            rope_scaling=scaling, max_position_embeddings=max_pos, tie_word_embeddings=tie,
            attention_bias=attn_bias, hidden_act=act, torch_dtype=dtype, bos_token_id=bos,
            eos_token_ids=eos_ids, sliding_window=window, layer_types=ltypes,
            extra={k: v for k, v in d.items() if k not in known},
        )
        cfg.validate()
        return cfg

    @classmethod
    def from_json_file(cls, path: str) -> "LlamaConfig":
        return cls.from_dict(read_config_json(path))

    def validate(self) -> None:
        def bounded(name: str, v: int, hi: int = DIM_MAX) -> None:
            if v < 1 or v > hi:
                raise ConfigError(f"config.json: {name}={v} is outside [1, {hi}]")
        bounded("hidden_size", self.hidden_size)
        bounded("num_hidden_layers", self.num_hidden_layers, LAYERS_MAX)
        bounded("num_attention_heads", self.num_attention_heads)
        bounded("num_key_value_heads", self.num_key_value_heads)
        bounded("head_dim", self.head_dim)
        bounded("intermediate_size", self.intermediate_size)
        bounded("vocab_size", self.vocab_size, 1 << 30)
        bounded("max_position_embeddings", self.max_position_embeddings, 1 << 30)
        bounded("num_attention_heads*head_dim", self.q_dim)
        if self.num_key_value_heads > self.num_attention_heads:
            raise ConfigError("config.json: num_key_value_heads exceeds num_attention_heads")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError("config.json: num_attention_heads is not a multiple of num_key_value_heads")
        if self.head_dim % 2 != 0:
            raise ConfigError("config.json: head_dim must be even (rotation works on pairs)")
        if not (self.rms_norm_eps > 0.0) or self.rms_norm_eps > 1.0:
            raise ConfigError(f"config.json: rms_norm_eps={self.rms_norm_eps} is outside (0, 1]")
        if not (self.rope_theta > 0.0):
            raise ConfigError(f"config.json: rope_theta={self.rope_theta} must be positive")
        if self.sliding_window is not None and self.sliding_window < 1:
            raise ConfigError("config.json: sliding_window must be >= 1 or null")
        if self.layer_types is not None:
            if len(self.layer_types) != self.num_hidden_layers:
                raise ConfigError("config.json: layer_types must name every layer")
            if self.sliding_window is None and "sliding_attention" in self.layer_types:
                raise ConfigError("config.json: layer_types names a sliding layer but sliding_window is null")
        for t in self.eos_token_ids + ((self.bos_token_id,) if self.bos_token_id is not None else ()):
            if t < 0 or t >= self.vocab_size:
                raise ConfigError(f"config.json: special token id {t} is outside the vocabulary")

    # ---- writing (random-weights mode) ------------------------------------
    def to_dict(self) -> dict:
        d = {
            "architectures": [self.architecture],
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": None,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": self.attention_bias,
            "mlp_bias": False,
            "hidden_act": self.hidden_act,
            "torch_dtype": self.torch_dtype,
        }
        if self.rope_scaling is not None:
            rs = self.rope_scaling
            d["rope_scaling"] = {"rope_type": "linear", "factor": rs.factor} if rs.rope_type == "linear" else {
                "rope_type": rs.rope_type, "factor": rs.factor,
                "low_freq_factor": rs.low_freq_factor, "high_freq_factor": rs.high_freq_factor,
                "original_max_position_embeddings": rs.original_max_position_embeddings,
            }
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            d["eos_token_id"] = self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else list(self.eos_token_ids)
        if self.sliding_window is not None:
            d["sliding_window"] = self.sliding_window
        if self.layer_types is not None:
            d["layer_types"] = list(self.layer_types)
        d.update(self.extra)
        return d


def _typed(key: str, v: Any, kind):
    if kind is bool:
        if not isinstance(v, bool):
            raise ConfigError(f"config.json: '{key}' must be true or false")
        return v
    if kind is int:
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"config.json: '{key}' must be an integer, got {v!r}")
        return v
    if kind is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: '{key}' must be a number, got {v!r}")
        return float(v)
    if kind is str:
        if not isinstance(v, str):
            raise ConfigError(f"config.json: '{key}' must be a string, got {v!r}")
        return v
    raise TypeError(kind)
