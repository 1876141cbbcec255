"""The tensor-core route of ``Linear``: bfloat16 activations times a bfloat16 matrix on tcgen05."""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels

ENABLED = True         # (False sends every product to the float32 FMA kernel: a test may set it to bisect a difference)


class Pending:
    """A product whose sum over its K slices is still to be taken: float32 partial sums [splits][n][width] in a
    slab of the product's workspace, to be summed into `out` (plus the bias).  Whoever takes the sum -- ``finish``,
    or a kernel that does it in passing -- calls ``release`` afterwards; until then the slab is this product's
    alone, so a part may start another product before it finishes this one."""

    def __init__(self, sums: "kernels.PartialSums", bias: Optional[torch.Tensor], out: torch.Tensor, accumulate: bool):
        self.sums, self.partial, self.splits = sums, sums.partial, sums.splits
        self.bias, self.out, self.accumulate = bias, out, accumulate

    def release(self) -> None:
        self.sums.release()

    def finish(self) -> None:
        kernels.finish_plain(self.partial, self.splits, self.bias, self.out, self.accumulate)
        self.release()


def usable(lin, x, out, accumulate) -> bool:
    return ENABLED and lin.weight is not None and kernels.gemm_tc_supported(x, lin.weight, out)


def run(lin, x, out, accumulate, defer=False, act=kernels.ACT_NONE):
    epi = kernels.EPI_ADD if accumulate else kernels.EPI_STORE
    w, packed_rows = (lin.packed, lin.n_out) if lin.packed is not None else (lin.weight, None)
    if defer:
        assert act == kernels.ACT_NONE
        sums = kernels.gemm_tc_deferred(x, w, out, lin.bias, epi, packed_rows=packed_rows)
        if sums is None:
            return None
        return Pending(sums, lin.bias, out, accumulate)
    kernels.gemm_tc(x, w, out, lin.bias, epi, packed_rows=packed_rows, act=act)
    return None
