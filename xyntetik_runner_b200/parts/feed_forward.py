"""Gated feed-forward: x += W_down . (silu(W_gate . h) * W_up . h), no biases
(src/model.c:6399-6407, 6421-6423; activation src/model.c:4451-4452)."""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import FeedForward, register_feed_forward
from .linear import Linear


class SwiGLU(FeedForward):
    graph_safe = True
    def __init__(self, width: int, inner: int, prefix: str,
                 gate: str = "gate_proj.weight", up: str = "up_proj.weight", down: str = "down_proj.weight"):
        self.width, self.inner, self.prefix = width, inner, prefix
        self.names = (prefix + gate, prefix + up, prefix + down)
        self.gate_up = self.down = None

    def tensors(self):
        g, u, d = self.names
        return {g: TensorSpec((self.inner, self.width)), u: TensorSpec((self.inner, self.width)),
                d: TensorSpec((self.width, self.inner))}

    def bind(self, tensors, rt):
        g, u, d = self.names
        wg, wu = tensors.pop(g), tensors.pop(u)
        if wg.dtype != wu.dtype:
            wg, wu = wg.to(torch.float32), wu.to(torch.float32)
        # one product for gate and up: rows [0, F) are the gate, [F, 2F) the up projection
        self.gate_up = Linear(torch.cat([wg, wu], dim=0), halves=2).prepare(rt)
        del wg, wu
        self.down = Linear(tensors[d]).prepare(rt)

    def weight_bytes(self):
        return self.gate_up.nbytes() + self.down.nbytes()

    def forward(self, ctx, h, x):
        n = h.shape[0]
        act = ctx.buf("ffn_act", (n, self.inner), ctx.act_dtype)
        if self.gate_up.swiglu_fused():
            # gate and up share the X tile; silu(g) * u happens in the product's epilogue
            self.gate_up.forward_swiglu(h, act)
        else:
            gu = ctx.buf("ffn_gate_up", (n, 2 * self.inner), ctx.act_dtype)
            self.gate_up.forward(h, gu)
            kernels.silu_mul(gu, act)
        ctx.set_pending(x, self.down.forward(act, x, accumulate=True, defer=True))


register_feed_forward("swiglu", SwiGLU)
