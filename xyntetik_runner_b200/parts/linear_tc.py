"""The tensor-core route of ``Linear``: bfloat16 activations times a bfloat16 matrix on tcgen05."""
from __future__ import annotations

import os

from .. import kernels

# XRB200_NO_TC=1 sends every product to the float32 FMA kernel (for bisecting a difference)
ENABLED = os.environ.get("XRB200_NO_TC", "0") in ("", "0")


def usable(lin, x, out, accumulate) -> bool:
    return ENABLED and kernels.gemm_tc_supported(x, lin.weight, out)


def run(lin, x, out, accumulate) -> None:
    kernels.gemm_tc(x, lin.weight, out, lin.bias, kernels.EPI_ADD if accumulate else kernels.EPI_STORE)
