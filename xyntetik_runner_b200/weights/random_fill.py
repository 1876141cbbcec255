"""Seeded normal values whose bits do not depend on where they are drawn.

``normal_values(key, first, count, mean, std)`` is a counter-based generator: value i is a function of
(key, first + i) alone, so a tensor can be drawn whole or in pieces, here with numpy or on the device by
``csrc/random_fill.cu`` (``kernels.random_normal``), and holds the same bits every time.  Both follow the
same recipe, in which every step is integer arithmetic or one correctly rounded float32 operation:

    h     = mix64(key + (index + 1) * 0x9E3779B97F4A7C15)          (the splitmix64 finaliser)
    u     = (2 * (h >> 41) + 1) * 2^-24                             in (0, 1), exact
    phase = (h >> 8) & 0xFFFFFF                                     24-bit fraction of a full turn
    z     = sqrt(-2 ln u) * cos(2 pi phase / 2^24)                  (Box-Muller)

with ln and cos from short float32 series (see the CUDA file for the decomposition).  The reference has
the same idea for its fixture only: an integer generator that anyone can run again
(scripts/make-test-model.py:238-252).
"""
from __future__ import annotations

import hashlib

import numpy as np

_U64 = np.uint64
_F = np.float32
_GOLD = _U64(0x9E3779B97F4A7C15)
_M1 = _U64(0xBF58476D1CE4E5B9)
_M2 = _U64(0x94D049BB133111EB)
# constants: doubles rounded once to float32, as in the CUDA file
_SQRT2, _INV_SQRT2, _LN2 = _F(1.4142135623730951), _F(0.7071067811865476), _F(0.6931471805599453)
_QUARTER_STEP = _F(1.5707963267948966 / 4194304.0)
_LN_C = [_F(1.0 / 9.0), _F(1.0 / 7.0), _F(1.0 / 5.0), _F(1.0 / 3.0), _F(1.0)]
_SIN_C = [_F(1.0 / 362880.0), _F(-1.0 / 5040.0), _F(1.0 / 120.0), _F(-1.0 / 6.0), _F(1.0)]
_COS_C = [_F(1.0 / 40320.0), _F(-1.0 / 720.0), _F(1.0 / 24.0), _F(-0.5), _F(1.0)]


def tensor_key(seed: int, name: str) -> int:
    """64-bit key of one tensor's values: every tensor draws independently of the others and of their sizes."""
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little")


def _mix64(z: np.ndarray) -> np.ndarray:
    z = (z ^ (z >> _U64(30))) * _M1
    z = (z ^ (z >> _U64(27))) * _M2
    return z ^ (z >> _U64(31))


def _poly(x: np.ndarray, coeff) -> np.ndarray:
    p = np.full_like(x, coeff[0])
    for c in coeff[1:]:
        p = p * x + c              # two float32 operations, two roundings (numpy does not fuse them)
    return p


def unit_normal_at(key: int, index: np.ndarray) -> np.ndarray:
    """z(key, index) in float32 for an array of element indices (uint64 or anything that converts)."""
    idx = np.asarray(index).astype(_U64)
    with np.errstate(over="ignore"):
        h = _mix64(_U64(key & 0xFFFFFFFFFFFFFFFF) + (idx + _U64(1)) * _GOLD)
    a = (h >> _U64(41)).astype(np.int64)
    u = (2 * a + 1).astype(_F) * _F(1.0 / 16777216.0)
    bits = u.view(np.uint32)
    e = (bits >> np.uint32(23)).astype(np.int32) - 127
    m = ((bits & np.uint32(0x7FFFFF)) | np.uint32(0x3F800000)).view(_F)
    big = m > _SQRT2
    m = np.where(big, m * _F(0.5), m)
    e = e + big.astype(np.int32)
    s = (m + _F(-1.0)) / (m + _F(1.0))
    s2 = s * s
    ln_m = (_F(2.0) * s) * _poly(s2, _LN_C)
    ln_u = e.astype(_F) * _LN2 + ln_m
    r = np.sqrt(_F(-2.0) * ln_u)
    b = ((h >> _U64(8)) & _U64(0xFFFFFF)).astype(np.int64)
    q = b >> 22
    w = (b & 0x3FFFFF) - (1 << 21)
    x = w.astype(_F) * _QUARTER_STEP
    x2 = x * x
    sx = x * _poly(x2, _SIN_C)
    cx = _poly(x2, _COS_C)
    s1 = (sx + cx) * _INV_SQRT2
    c1 = (cx + (-sx)) * _INV_SQRT2
    c = np.where(q == 0, c1, np.where(q == 1, -s1, np.where(q == 2, -c1, s1)))
    out = r * c
    assert out.dtype == _F
    return out


def normal_values(key: int, first: int, count: int, mean: float, std: float) -> np.ndarray:
    """mean + std * z(key, first + i) for i in [0, count), float32, drawn in pieces of a few million."""
    out = np.empty(count, dtype=_F)
    step = 1 << 22
    for at in range(0, count, step):
        n = min(step, count - at)
        z = unit_normal_at(key, np.arange(first + at, first + at + n, dtype=_U64))
        out[at:at + n] = _F(mean) + z * _F(std)
    return out


def to_bfloat16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> the 16 bits of the nearest bfloat16 (ties to even), as uint16."""
    b = np.ascontiguousarray(x, dtype=_F).view(np.uint32)
    return ((b + np.uint32(0x7FFF) + ((b >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)
