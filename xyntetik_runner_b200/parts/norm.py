"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, computed in float32 (src/model.c:3386-3392)."""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import Norm, register_norm


class RMSNorm(Norm):
    graph_safe = True
    def __init__(self, width: int, eps: float, name: str):
        self.width, self.eps, self.name = width, float(eps), name
        self.weight = None

    def tensors(self):
        return {self.name: TensorSpec((self.width,), kind="vector", init="ones_jitter")}

    def bind(self, tensors, rt):
        # norm weights are used in float32 whatever they were stored in (src/model.c:2830-2831)
        self.weight = tensors[self.name].to(torch.float32).contiguous()

    def weight_bytes(self):
        return self.width * 4

    def forward(self, ctx, x, out, rows=None):
        pend = ctx.take_pending(x)
        if pend is not None and rows is None:
            # the product before this norm left partial sums: sum, add into x and normalise in one pass
            kernels.finish_add_rmsnorm(pend.partial, pend.splits, pend.bias, x, self.weight, out, self.eps)
            pend.release()
            return
        if pend is not None:
            pend.finish()
        kernels.rmsnorm(x, self.weight, out, self.eps, rows)


register_norm("rmsnorm", RMSNorm)
