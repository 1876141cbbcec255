"""A weight matrix and the choice of kernel that multiplies by it.

``out[t][r] (+)= sum_k x[t][k] W[r][k] (+ bias[r])``.  W keeps its stored dtype.  bfloat16 activations times
a bfloat16 matrix go to the tensor-core kernel (tcgen05); for that the matrix is re-laid tile by tile when the
part binds it (``prepare``), so that every tile the kernel streams is one contiguous read.  Everything else
-- the true 32-bit path above all -- goes to the float32 FMA kernel on the matrix as stored.  Which kernel
ran is counted, so that a test can prove its subject ran.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from . import linear_tc

counters = {"tcgen05": 0, "simt": 0, "deferred": 0}


class Linear:
    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, halves: int = 1):
        """`halves` = 2: the rows are two matrices of equal height (gate, up) that the tensor-core kernel
        multiplies side by side (see ``forward_swiglu``)."""
        assert weight.dim() == 2 and weight.shape[0] % halves == 0
        self.weight: Optional[torch.Tensor] = weight.contiguous()
        self.bias = None if bias is None else bias.to(torch.float32).contiguous()
        self.n_out, self.k = self.weight.shape
        self.halves = halves
        self.packed: Optional[torch.Tensor] = None
        self._nbytes = self.weight.numel() * self.weight.element_size()

    def prepare(self, rt, keep_plain: bool = False) -> "Linear":
        """Choose the layout for the engine's precision.  Returns self."""
        if (linear_tc.ENABLED and rt.act_dtype == torch.bfloat16 and self.weight.dtype == torch.bfloat16
                and self.k % 8 == 0 and self.weight.is_cuda):
            self.packed = kernels.pack_weight(self.weight, self.halves)
            if not keep_plain:
                self.weight = None
        return self

    def nbytes(self) -> int:
        return self._nbytes

    def forward(self, x: torch.Tensor, out: torch.Tensor, accumulate: bool = False, defer: bool = False,
                act: int = kernels.ACT_NONE):
        """out (+)= act(x W^T + bias) (an activation only without `accumulate`).  With `defer`, a product that was
        split along K leaves its partial sums in a slab of the workspace and returns ``Pending``; the caller's next
        kernel sums them (and adds the bias) and releases the slab.  Otherwise returns None and `out` is complete."""
        assert self.halves == 1, "a matrix of two halves is multiplied by forward_gated"
        assert act == kernels.ACT_NONE or not (accumulate or defer)
        if self.packed is not None or linear_tc.usable(self, x, out, accumulate):
            counters["tcgen05"] += 1
            pending = linear_tc.run(self, x, out, accumulate, defer, act)
            if pending is not None:
                counters["deferred"] += 1
            return pending
        kernels.gemm_simt(x, self.weight, out, self.bias, accumulate)
        if act != kernels.ACT_NONE:
            kernels.act_mul(out, out, act, gated=False)
        counters["simt"] += 1
        return None

    def gated_fused(self) -> bool:
        return self.halves == 2 and self.packed is not None

    def forward_gated(self, x: torch.Tensor, out: torch.Tensor, act: int = kernels.ACT_SILU,
                      scratch: Optional[torch.Tensor] = None) -> None:
        """out[t][f] = act(x . W_gate[f]) * (x . W_up[f]): in the tensor-core product's epilogue when the matrix is
        packed for it, else as the product [n, 2F] into `scratch` followed by the activation kernel."""
        assert self.halves == 2
        if self.packed is not None:
            kernels.gemm_tc(x, self.packed, out, None, kernels.EPI_GATED, packed_rows=self.n_out // 2, act=act)
            counters["tcgen05"] += 1
            return
        assert scratch is not None and scratch.shape == (x.shape[0], self.n_out)
        kernels.gemm_simt(x, self.weight, scratch, None, False)
        counters["simt"] += 1
        kernels.act_mul(scratch, out, act, gated=True)
