"""The tensor-core route of ``Linear``: bfloat16 activations times a bfloat16 matrix on tcgen05."""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch

from .. import kernels

# XRB200_NO_TC=1 sends every product to the float32 FMA kernel (for bisecting a difference)
ENABLED = os.environ.get("XRB200_NO_TC", "0") in ("", "0")


@dataclass
class Pending:
    """Partial sums [splits][n][width] float32 of a product that still have to be summed into `out`."""
    partial: torch.Tensor
    splits: int
    bias: Optional[torch.Tensor]
    out: torch.Tensor
    accumulate: bool

    def finish(self) -> None:
        kernels.finish_plain(self.partial, self.splits, self.bias, self.out, self.accumulate)


def usable(lin, x, out, accumulate) -> bool:
    return ENABLED and lin.weight is not None and kernels.gemm_tc_supported(x, lin.weight, out)


def run(lin, x, out, accumulate, defer=False):
    epi = kernels.EPI_ADD if accumulate else kernels.EPI_STORE
    if lin.packed is not None:
        splits = kernels.gemm_tc(x, lin.packed, out, lin.bias, epi, defer=defer, packed_rows=lin.n_out)
    else:
        splits = kernels.gemm_tc(x, lin.weight, out, lin.bias, epi, defer=defer)
    if defer and splits > 1:
        return Pending(kernels.tc_workspace(x.device)[0], splits, lin.bias, out, accumulate)
    return None
