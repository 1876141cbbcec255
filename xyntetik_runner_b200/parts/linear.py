"""A weight matrix and the choice of kernel that multiplies by it.

``out[t][r] (+)= sum_k x[t][k] W[r][k] (+ bias[r])``.  W keeps its stored dtype.
bfloat16 activations times a bfloat16 matrix go to the tensor-core kernel
(tcgen05, when the shapes meet its alignment rules); everything else -- the
true 32-bit path above all -- goes to the float32 FMA kernel.  Which kernel ran
is counted, so that a test can prove its subject ran.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels

counters = {"tcgen05": 0, "simt": 0}


class Linear:
    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        assert weight.dim() == 2
        self.weight = weight.contiguous()
        self.bias = None if bias is None else bias.to(torch.float32).contiguous()
        self.n_out, self.k = self.weight.shape
        self._tc = None          # tensor-core plan (built on first use)

    def nbytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, x: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
        from . import linear_tc
        if linear_tc.usable(self, x, out, accumulate):
            linear_tc.run(self, x, out, accumulate)
            counters["tcgen05"] += 1
        else:
            kernels.gemm_simt(x, self.weight, out, self.bias, accumulate)
            counters["simt"] += 1
