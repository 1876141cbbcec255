"""Feed-forwards.  Gated: x += W_down . (act(W_gate . h) * W_up . h); ungated: x += W_down . act(W_up . h); no biases
(src/model.c:6378-6423; activations src/model.c:4425-4452: SiLU for the llama family, tanh-GELU for others)."""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import FeedForward, register_feed_forward
from .linear import Linear


def _act_id(activation: str) -> int:
    try:
        return kernels.ACTIVATIONS[activation]
    except KeyError:
        raise ValueError(f"activation '{activation}': known are {sorted(kernels.ACTIVATIONS)}") from None


class GatedFeedForward(FeedForward):
    """act(gate) * up, then down.  `activation` "silu" is SwiGLU."""
    graph_safe = True

    def __init__(self, width: int, inner: int, prefix: str, activation: str = "silu",
                 gate: str = "gate_proj.weight", up: str = "up_proj.weight", down: str = "down_proj.weight"):
        self.width, self.inner, self.prefix = width, inner, prefix
        self.act = _act_id(activation)
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
        # gate and up share the X tile; act(g) * u happens in the product's epilogue where the tensor cores run it
        gu = None if self.gate_up.gated_fused() else ctx.buf("ffn_gate_up", (n, 2 * self.inner), ctx.act_dtype)
        self.gate_up.forward_gated(h, act, self.act, gu)
        ctx.set_pending(x, self.down.forward(act, x, accumulate=True, defer=True))


class SwiGLU(GatedFeedForward):
    def __init__(self, width: int, inner: int, prefix: str, **names):
        super().__init__(width, inner, prefix, "silu", **names)


class MLP(FeedForward):
    """Ungated: x += W_down . act(W_up . h)."""
    graph_safe = True

    def __init__(self, width: int, inner: int, prefix: str, activation: str = "gelu_tanh",
                 up: str = "up_proj.weight", down: str = "down_proj.weight"):
        self.width, self.inner, self.prefix = width, inner, prefix
        self.act = _act_id(activation)
        self.names = (prefix + up, prefix + down)
        self.up = self.down = None

    def tensors(self):
        u, d = self.names
        return {u: TensorSpec((self.inner, self.width)), d: TensorSpec((self.width, self.inner))}

    def bind(self, tensors, rt):
        u, d = self.names
        self.up = Linear(tensors[u]).prepare(rt)
        self.down = Linear(tensors[d]).prepare(rt)

    def weight_bytes(self):
        return self.up.nbytes() + self.down.nbytes()

    def forward(self, ctx, h, x):
        act = ctx.buf("ffn_act", (h.shape[0], self.inner), ctx.act_dtype)
        self.up.forward(h, act, act=self.act)          # the activation rides in the product's epilogue
        ctx.set_pending(x, self.down.forward(act, x, accumulate=True, defer=True))


register_feed_forward("swiglu", SwiGLU)
register_feed_forward("gated", GatedFeedForward)
register_feed_forward("mlp", MLP)
