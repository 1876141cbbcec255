"""Position encodings.  Rotary: per-pair frequencies built once in float32.

inv_freq[j] = theta^(-2j / rotary_dim) (float32 `powf`, src/model.c:288-289), divided by the
model's per-frequency factors where it has them (src/model.c:291-297).  The reference reads those
factors from a tensor its converter wrote; for ``rope_scaling`` of type llama3 they are computed
here from the four numbers of the configuration: with wavelength lam = 2*pi/f,
``lam < orig/high`` keeps f, ``lam > orig/low`` divides f by ``factor``, and between the two
f' = (1-s) f/factor + s f with s = (orig/lam - low) / (high - low).  ``rope_scaling`` of type linear divides
every frequency by ``factor`` (src/model.c:361-362).  The rotation itself (angle =
position * inv_freq in float32, pairs (j, j + rotary_dim/2), src/model.c:3514-3532) happens in the
kernel that also stores K and V.
"""
from __future__ import annotations

import math
from typing import Optional

import numpy as np
import torch

from .base import PositionEncoding, Rotary, register_position


def llama3_divisors(inv_freq: np.ndarray, factor: float, low: float, high: float, orig: int) -> np.ndarray:
    out = np.ones_like(inv_freq, dtype=np.float32)
    for j, f in enumerate(inv_freq.tolist()):
        lam = 2.0 * math.pi / f
        if lam < orig / high:
            d = 1.0
        elif lam > orig / low:
            d = factor
        else:
            s = (orig / lam - low) / (high - low)
            d = f / ((1.0 - s) * f / factor + s * f)
        out[j] = np.float32(d)
    return out


class Rope(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, rotary_dim: Optional[int] = None, scaling=None,
                 pairing: str = "half", mscale: float = 1.0):
        """pairing "half" rotates elements (j, j + rotary_dim/2), the layout of a config.json + safetensors
        checkpoint; "adjacent" rotates (2j, 2j + 1), the layout the reference's llama files carry
        (src/model.c:1464-1466).  mscale multiplies every cosine and sine (src/model.c:283, 375)."""
        self.head_dim = head_dim
        self.pairing, self.mscale = pairing, float(mscale)
        self.rotary_dim = head_dim if rotary_dim is None else rotary_dim
        if self.rotary_dim % 2 or self.rotary_dim > head_dim or self.rotary_dim < 0:
            raise ValueError("rotary_dim must be even and at most head_dim")
        half = self.rotary_dim // 2
        j = np.arange(half, dtype=np.float32)
        expo = (np.float32(-2.0) * j / np.float32(self.rotary_dim)).astype(np.float32) if half else j
        inv = np.power(np.float32(theta), expo).astype(np.float32)
        if scaling is not None and getattr(scaling, "rope_type", "llama3") == "linear":
            inv = (inv / np.float32(scaling.factor)).astype(np.float32)          # src/model.c:361-362
        elif scaling is not None:
            div = llama3_divisors(inv, scaling.factor, scaling.low_freq_factor, scaling.high_freq_factor,
                                  scaling.original_max_position_embeddings)
            inv = (inv / div).astype(np.float32)
        self.inv_freq_host = inv
        self.inv_freq = None

    def prepare(self, rt):
        self.inv_freq = torch.from_numpy(self.inv_freq_host.copy()).to(rt.device)

    def rotary(self):
        return Rotary(self.rotary_dim, self.inv_freq if self.rotary_dim else None, self.pairing, self.mscale)


class NoPosition(PositionEncoding):
    """No position signal of its own (order comes from the causal mask alone)."""

    def rotary(self):
        return None


register_position("rope", Rope)
register_position("none", NoPosition)
