"""The tensor-core route of ``Linear`` (filled in by the tcgen05 kernel's wrapper)."""
from __future__ import annotations

ENABLED = False


def usable(lin, x, out, accumulate) -> bool:
    return False


def run(lin, x, out, accumulate) -> None:
    raise RuntimeError("tensor-core product is not available")
