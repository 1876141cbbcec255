"""Python face of the CUDA library: one function per launcher, torch tensors in.

Every function checks what the kernel cannot (device, dtype, contiguity),
launches on torch's current stream and raises on a refusal.  Nothing here has
another way to compute its result: if the library cannot be built or loaded,
the first call raises.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
_ERR = {-1: "the kernel refuses these sizes or dtypes", -2: "CUDA refused the launch", -3: "tensor map encoding failed",
        -4: "size beyond the entry point's fixed limit", -5: "set-up of the entry point failed"}

_lib = None


class KernelError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = _build.library_path()
        try:
            _lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load {path}: {e}") from None
        _declare(_lib)
    return _lib


def library_file() -> str:
    lib()
    return _build.library_path(build=False)


_vp, _i, _ll, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


def _declare(L: ctypes.CDLL) -> None:
    sig = {
        "xr_embed": [_vp, _i, _vp, _vp, _i, _vp, _i, _i, _i, _vp],
        "xr_rmsnorm": [_vp, _vp, _vp, _vp, _i, _i, _i, _f, _vp],
        "xr_rope_store": [_vp, _i, _vp, _vp, _vp, _vp, _vp, _ll, _ll, _i, _i, _i, _i, _i, _i, _i, _i, _f, _vp],
        "xr_act_mul": [_vp, _vp, _i, _i, _i, _i, _i, _vp],
        "xr_residual_add": [_vp, _vp, _i, _i, _i, _vp],
        "xr_gemm_simt": [_vp, _i, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _ll, _ll, _vp],
        "xr_attention_simt": [_vp, _vp, _i, _vp, _vp, _vp, _vp, _ll, _ll, _ll, _i, _i, _i, _i, _i, _i, _i, _f, _vp],
        "xr_gemm_tc": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _ll, _ll, _vp, _ll, _vp, _i, _i, ctypes.POINTER(ctypes.c_int), _i, _vp],
        "xr_finish_add_rmsnorm": [_vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _vp],
        "xr_finish_plain": [_vp, _i, _vp, _vp, _i, _i, _i, _i, _ll, _vp],
        "xr_finish_rope_store": [_vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _ll, _i, _i, _i, _i, _i, _i, _i, _i, _f, _vp],
        "xr_attention_mma": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _ll, _ll, _i, _i, _i, _i, _i, _i, _i, _f,
                             _i, _i, _i, _i, _i, _vp, _ll, _i, _i, _vp, _vp, _i, _i, _ll, _vp],
        "xr_attention_mma_splits": [_i, _i, _ll],
        "xr_attention_even_launches": [],
        "xr_attention_wait_probe": [_vp, _vp, ctypes.c_uint, _vp],
        "xr_attention_tc_supported": [_i, _i, _i, _i],
        "xr_attention_tc": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _ll, _ll, _i, _i, _vp],
        "xr_sample": [_vp, _ll, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp],
        "xr_sample_one_block": [_vp, _ll, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
        "xr_logprob": [_vp, _ll, _i, _i, _vp, _vp, _vp],
        "xr_random_normal": [_vp, _i, _ll, ctypes.c_ulonglong, ctypes.c_ulonglong, _f, _f, _vp],
    }
    for name, args in sig.items():
        fn = getattr(L, name)
        fn.argtypes = args
        fn.restype = ctypes.c_int


def _check(code: int, what: str) -> None:
    if code != 0:
        raise KernelError(f"{what}: {_ERR.get(code, f'error {code}')}")


try:
    _raw_stream, _raw_device = torch._C._cuda_getCurrentRawStream, torch._C._cuda_getDevice
except AttributeError:                   # (another torch: the documented way, a few microseconds a call)
    _raw_stream = _raw_device = None


def _stream() -> int:
    """The current CUDA stream's handle.  Asked for at every launch: a step of a few hundred tokens is a few hundred
    launches whose host time nothing hides, so it is the two C calls, not the Stream object that torch builds."""
    if _raw_stream is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"dtype {dt} is not float32 or bfloat16")


def _dev(*ts) -> None:
    for t in ts:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise KernelError("kernel arguments must be contiguous CUDA tensors")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


launch_count = 0   # kernels launched through this module since import (bench reports it)


def _count(n: int = 1) -> None:
    global launch_count
    launch_count += n


# ---------------------------------------------------------------------------
def embed(table: torch.Tensor, ids: torch.Tensor, x: torch.Tensor, feed: Optional[torch.Tensor] = None) -> None:
    """x[t] = table[ids[t]] widened to float32; ids outside the table read row 0.  With `feed` (int32 on the
    device), ids[t] = -(1 + j) reads token feed[j]."""
    _dev(table, ids, x, feed)
    n, d = x.shape
    assert ids.dtype == torch.int32 and ids.numel() >= n and x.dtype == torch.float32 and table.shape[1] == d
    assert feed is None or feed.dtype == torch.int32
    _check(lib().xr_embed(table.data_ptr(), dtype_code(table.dtype), ids.data_ptr(), _ptr(feed),
                          0 if feed is None else feed.numel(), x.data_ptr(), n, d, table.shape[0], _stream()), "embed")
    _count()


def rmsnorm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, eps: float, rows: Optional[torch.Tensor] = None) -> None:
    """out[i] = x[rows[i] or i] * rsqrt(mean(x^2) + eps) * w; x float32, w float32."""
    _dev(x, w, out, rows)
    n, d = out.shape
    assert x.dtype == torch.float32 and w.dtype == torch.float32 and x.shape[1] == d and w.numel() == d
    assert rows is None or (rows.dtype == torch.int32 and rows.numel() >= n)
    _check(lib().xr_rmsnorm(x.data_ptr(), _ptr(rows), w.data_ptr(), out.data_ptr(), dtype_code(out.dtype), n, d,
                            float(eps), _stream()), "rmsnorm")
    _count()


def rope_store(qkv: torch.Tensor, positions, tok_seg, block_tables, inv_freq: Optional[torch.Tensor],
               cache_k_ptr: Optional[int], page_stride: int, v_offset: int, H: int, K: int, hd: int,
               rotary_dim: int, max_pages: int, page_size: int, adjacent: bool = False, mscale: float = 1.0) -> None:
    """Rotate Q in place, rotate K and store K, V into their pages (cache_k_ptr None: store nothing).  Pair j of
    a head is elements (j, j + rotary_dim/2), or (2j, 2j + 1) with `adjacent`; cosines and sines are multiplied
    by `mscale` (src/model.c:3514-3532)."""
    _dev(qkv, positions, tok_seg, block_tables, inv_freq)
    n = qkv.shape[0]
    assert qkv.shape[1] == (H + 2 * K) * hd
    assert rotary_dim == 0 or (inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() >= rotary_dim // 2)
    _check(lib().xr_rope_store(qkv.data_ptr(), dtype_code(qkv.dtype), positions.data_ptr(), tok_seg.data_ptr(),
                               block_tables.data_ptr(), _ptr(inv_freq), cache_k_ptr, page_stride, v_offset,
                               n, H, K, hd, rotary_dim, max_pages, page_size, int(adjacent), float(mscale), _stream()),
           "rope_store")
    _count()


ACT_NONE, ACT_SILU, ACT_GELU_TANH = 0, 1, 2
ACTIVATIONS = {"none": ACT_NONE, "silu": ACT_SILU, "gelu_tanh": ACT_GELU_TANH}


def act_mul(gu: torch.Tensor, h: torch.Tensor, act: int = ACT_SILU, gated: bool = True) -> None:
    """Gated: h[t][f] = act(gu[t][f]) * gu[t][F + f] for gu [n, 2F]; ungated: h = act(gu) for gu [n, F] (h may be gu)."""
    _dev(gu, h)
    n, F = h.shape
    assert gu.shape == (n, 2 * F if gated else F) and gu.dtype == h.dtype
    _check(lib().xr_act_mul(gu.data_ptr(), h.data_ptr(), dtype_code(h.dtype), n, F, int(act), int(gated), _stream()), "act_mul")
    _count()


def silu_mul(gu: torch.Tensor, h: torch.Tensor) -> None:
    act_mul(gu, h, ACT_SILU, True)


def residual_add(x: torch.Tensor, delta: torch.Tensor) -> None:
    _dev(x, delta)
    n, d = x.shape
    assert x.dtype == torch.float32 and delta.shape == x.shape
    _check(lib().xr_residual_add(x.data_ptr(), delta.data_ptr(), dtype_code(delta.dtype), n, d, _stream()), "residual_add")
    _count()


def gemm_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
              accumulate: bool = False) -> None:
    """out[t][r] (+)= sum_k x[t][k] w[r][k] (+ bias[r]) in float32 FMA.  Rows of x and out may be strided."""
    for t in (x, w, out, bias):
        if t is not None and not t.is_cuda:
            raise KernelError("kernel arguments must be CUDA tensors")
    n, k = x.shape
    n_out = w.shape[0]
    assert w.shape[1] == k and out.shape == (n, n_out) and w.is_contiguous()
    assert x.stride(1) == 1 and out.stride(1) == 1
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == n_out)
    _check(lib().xr_gemm_simt(x.data_ptr(), dtype_code(x.dtype), w.data_ptr(), dtype_code(w.dtype), _ptr(bias),
                              out.data_ptr(), dtype_code(out.dtype), int(accumulate), n, n_out, k,
                              x.stride(0), out.stride(0), _stream()), "gemm_simt")
    _count()


def attention_simt(q: torch.Tensor, q_row_stride: int, out: torch.Tensor, cache_k_ptr: int, positions, tok_seg,
                   block_tables, page_stride: int, v_offset: int, H: int, K: int, hd: int, max_pages: int,
                   page_size: int, window: int, scale: float) -> None:
    """Causal attention of every token of the step over its request's pages, float32 arithmetic."""
    _dev(out, positions, tok_seg, block_tables)
    n = out.shape[0]
    assert out.shape[1] == H * hd and q.dtype == out.dtype
    _check(lib().xr_attention_simt(q.data_ptr(), out.data_ptr(), dtype_code(out.dtype), cache_k_ptr,
                                   positions.data_ptr(), tok_seg.data_ptr(), block_tables.data_ptr(), page_stride,
                                   v_offset, q_row_stride, n, H, K, hd, max_pages, page_size, window, float(scale),
                                   _stream()), "attention_simt")
    _count()


EXEMPT_IDS = 8          # ids per row that a penalty window never holds, as the sampling kernel takes them


def sample(logits: torch.Tensor, temp, top_k, top_p, min_p, penalty, draw, recent: Optional[torch.Tensor],
           scratch: torch.Tensor, out: torch.Tensor, any_sampled: bool = True, one_block: bool = False,
           shortcuts: bool = True, pending: Optional[torch.Tensor] = None, feed: Optional[torch.Tensor] = None,
           exempt: Optional[torch.Tensor] = None) -> None:
    """One token per row of float32 logits by the reference's sampling chain (see csrc/sampling.cu).
    `scratch` must hold rows * vocab floats unless every row is greedy (`any_sampled` False).  `shortcuts` (the
    default): one block a row that selects the top-k, or gathers the head of the distribution, sorts that and walks
    it as the reference does; rows where that does not apply are left to a second launch that goes the long way for
    them alone.  Without: the long way for every row, by threshold descents that never sort, spread over a cluster of
    eight blocks a row when the rows are few and have more than 1,024 values (`one_block`: in one block whatever the width).
    `pending` (int32 [rows, 3]) with `feed` and `exempt` (int32 [rows, EXEMPT_IDS]): row r's window lacks the token that
    the step before sampled and the host has not read yet; it is feed[pending[r, 0]] (-1: the window is complete),
    takes window entry pending[r, 1], and is left out if it is among the first pending[r, 2] ids of exempt[r].
    `out` must not be `feed` then."""
    _dev(temp, top_k, top_p, min_p, penalty, draw, recent, scratch, out)
    rows, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert not any_sampled or scratch.numel() >= rows * V
    assert out.dtype == torch.int32 and top_k.dtype == torch.int32
    # (rows that are all greedy are one argmax each: nothing for a cluster to share)
    args = (logits.data_ptr(), logits.stride(0), rows, V, temp.data_ptr(), top_k.data_ptr(), top_p.data_ptr(), min_p.data_ptr(),
            penalty.data_ptr(), draw.data_ptr(), _ptr(recent), scratch.data_ptr(), out.data_ptr())
    if pending is not None:
        _dev(pending, feed, exempt)
        assert pending.dtype == torch.int32 and pending.numel() >= 3 * rows and exempt.dtype == torch.int32
        assert exempt.numel() >= EXEMPT_IDS * rows and feed.dtype == torch.int32 and recent is not None
        assert out.data_ptr() != feed.data_ptr() and any_sampled and not one_block
    if one_block or not any_sampled:
        _check(lib().xr_sample_one_block(*args, _stream()), "sample")
    else:
        _check(lib().xr_sample(*args, int(shortcuts), _ptr(pending), _ptr(feed), _ptr(exempt), _stream()), "sample")
    _count()


def logprob(logits: torch.Tensor, target: torch.Tensor, out: torch.Tensor) -> None:
    """out[i] = log softmax(logits[i])[target[i]] (float maximum, double sum of exponentials, float result)."""
    _dev(target, out)
    rows, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and logits.is_cuda
    assert target.dtype == torch.int32 and target.numel() >= rows and out.dtype == torch.float32 and out.numel() >= rows
    _check(lib().xr_logprob(logits.data_ptr(), logits.stride(0), rows, V, target.data_ptr(), out.data_ptr(), _stream()), "logprob")
    _count()


def random_normal(out: torch.Tensor, key: int, mean: float, std: float, first: int = 0) -> None:
    """out.flat[i] = mean + std * z(key, first + i): the counter-based generator of csrc/random_fill.cu, whose
    values equal ``weights.random_fill.normal_values`` bit for bit."""
    _dev(out)
    _check(lib().xr_random_normal(out.data_ptr(), dtype_code(out.dtype), out.numel(), key & 0xFFFFFFFFFFFFFFFF, first,
                                  float(mean), float(std), _stream()), "random_normal")
    _count()


# ---------------------------------------------------------------------------
EPI_STORE, EPI_ADD, EPI_GATED = 0, 1, 2
EPI_SWIGLU = EPI_GATED          # the gated epilogue with the SiLU activation
_TC_SCRATCH_FLOATS = 32 << 20
_HANDOVER_FLAGS = 2048          # one word per CTA of the decode attention in even shares
_tc_state = {}


class Workspace:
    """Split-K scratch and status word of the tensor-core product on one device.

    A product that is cut along K leaves float32 partial sums here.  When its caller defers the sum to its next
    kernel the slab stays taken until that kernel has been launched (``PartialSums.release``), and products
    launched meanwhile get room behind it: two deferred sums can never share memory, whatever order a block
    runs its parts in.  Slabs are handed out by a bump pointer that returns to the start whenever nothing is
    outstanding, so the usual order (product, then the kernel that sums it) always uses the same addresses,
    which CUDA graphs need.  ``reset`` (called at the start of every engine step) drops slabs that a failed
    step left behind."""

    def __init__(self, device: torch.device):
        self.scratch = torch.empty(_TC_SCRATCH_FLOATS, dtype=torch.float32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.status_ptr = self.status.data_ptr()
        self.flags = torch.zeros(_HANDOVER_FLAGS, dtype=torch.int32, device=device)   # raised and lowered inside one launch
        self.top = 0            # floats taken from the start of the scratch
        self.live = 0           # slabs outstanding

    def reset(self) -> None:
        self.top = self.live = 0

    def room(self):
        """(address, floats) of the free part."""
        if self.live == 0:
            self.top = 0
        return self.scratch.data_ptr() + 4 * self.top, self.scratch.numel() - self.top

    def take(self, floats: int) -> torch.Tensor:
        at = self.top
        self.top += (floats + 63) // 64 * 64
        self.live += 1
        return self.scratch[at:at + floats]

    def give_back(self) -> None:
        self.live = max(0, self.live - 1)
        if self.live == 0:
            self.top = 0


def workspace(device: torch.device) -> Workspace:
    key = device.index if device.index is not None else torch.cuda.current_device()
    ws = _tc_state.get(key)
    if ws is None:
        ws = _tc_state[key] = Workspace(device)
    return ws


def tc_workspace(device: torch.device):
    """(split-K scratch, status word) of the tensor-core product on `device`, made on first use."""
    ws = workspace(device)
    return ws.scratch, ws.status


def tc_workspace_reset(device: torch.device) -> None:
    """Forget deferred sums that were never finished (a step that failed half way)."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key in _tc_state:
        _tc_state[key].reset()


def tc_check_status(device: torch.device) -> None:
    """Raise if a tensor-core kernel gave up a wait since the last check (reads one word from the device)."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    ws = _tc_state.get(key)
    if ws is not None:
        code = int(ws.status.item())
        if code != 0:
            ws.status.zero_()
            ws.flags.zero_()                  # a launch that gave up may have left some raised
            what = {1: "a tcgen05 product", 2: "the bulk-copy decode attention", 3: "the tcgen05 attention", 4: "the tcgen05 attention (shared memory not 1 KB aligned)"}.get(code, "a kernel")
            raise KernelError(f"{what} gave up waiting on a barrier; its output is not valid")


def gemm_tc_supported(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    k = x.shape[1]
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and k >= 8 and k % 8 == 0 and x.stride(1) == 1
            and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and w.is_contiguous()
            and out.stride(1) == 1)


TILE_ROWS, TILE_K = 128, 64
GATED_FEATURES = 64        # features per 128-row tile of a gated product


def pack_weight(w: torch.Tensor, halves: int = 1) -> torch.Tensor:
    """Re-lay a [rows, K] bfloat16 matrix tile by tile for the tensor-core product:
    [row tile][K block][128][64], rows and K padded with zeros to whole tiles, so that every tile the
    kernel fetches is one contiguous 16 KB read.

    `halves` = 2: the rows are F gate rows followed by F up rows of a gated product.  They are interleaved so that
    a 128-row tile holds 64 features: its rows 32 q .. 32 q + 15 are the gate rows of features 64 tile + 16 q + (0..15)
    and rows 32 q + 16 .. 32 q + 31 their up rows (q = 0..3: the four quarters of the accumulator's lanes), which
    lets the product's epilogue combine a feature's two sums inside one warp."""
    assert w.dtype == torch.bfloat16 and w.dim() == 2 and w.shape[0] % halves == 0 and halves in (1, 2)
    rows, k = w.shape[0] // halves, w.shape[1]
    kp = -(-k // TILE_K) * TILE_K
    if halves == 2:
        fp = -(-rows // GATED_FEATURES) * GATED_FEATURES
        both = torch.zeros((2, fp, kp), dtype=w.dtype, device=w.device)
        both[0, :rows, :k] = w[:rows]
        both[1, :rows, :k] = w[rows:]
        # [half][tile][quarter][16][K] -> [tile][quarter][half][16][K]
        src = both.view(2, fp // GATED_FEATURES, 4, 16, kp).permute(1, 2, 0, 3, 4).reshape(fp * 2, kp)
        del both
    else:
        rp = -(-rows // TILE_ROWS) * TILE_ROWS
        if rp != rows or kp != k:
            src = torch.zeros((rp, kp), dtype=w.dtype, device=w.device)
            src[:rows, :k] = w
        else:
            src = w
    rp = src.shape[0]
    return src.view(rp // TILE_ROWS, TILE_ROWS, kp // TILE_K, TILE_K).permute(0, 2, 1, 3).contiguous()


class PartialSums:
    """float32 partial sums [splits][n][rows] of a product that was cut along K and whose sum is left to the
    caller's next kernel.  The slab of the workspace they lie in is this object's until ``release``."""

    def __init__(self, ws: Workspace, partial: torch.Tensor, splits: int):
        self._ws, self.partial, self.splits = ws, partial, splits

    def release(self) -> None:
        if self._ws is not None:
            self._ws.give_back()
            self._ws = None


_SPLITS_USED = ctypes.c_int(1)           # where xr_gemm_tc says how it cut the product (read at once after the call)
_SPLITS_USED_REF = ctypes.byref(_SPLITS_USED)


def _gemm_tc(x, w, out, bias, epilogue, act, force_splits, defer, packed_rows):
    n, k = x.shape
    gated = epilogue == EPI_GATED
    if packed_rows is not None:
        # w comes from pack_weight(); packed_rows is the logical number of output features
        n_out = packed_rows
        tiles = -(-n_out // GATED_FEATURES) if gated else -(-n_out // TILE_ROWS)
        assert w.dim() == 4 and w.shape[0] == tiles and w.shape[1] == -(-k // TILE_K) and out.shape == (n, n_out)
        assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and k % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0
    else:
        if gated:
            raise KernelError("the gated product takes weights from pack_weight(w, halves=2)")
        n_out = w.shape[0]
        assert w.shape[1] == k and out.shape == (n, n_out) and gemm_tc_supported(x, w, out)
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == n_out and not gated)
    assert not defer or not gated
    ws = workspace(x.device)
    at, room = ws.room()
    _check(lib().xr_gemm_tc(x.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), dtype_code(out.dtype), epilogue, int(act),
                            n, n_out, k, x.stride(0), out.stride(0), at, room,
                            ws.status_ptr, force_splits, int(defer), _SPLITS_USED_REF,
                            int(packed_rows is not None), _stream()), "gemm_tc")
    splits = _SPLITS_USED.value
    _count(1 if (splits == 1 or defer) else 2)
    if defer and splits > 1:
        rows = tiles * TILE_ROWS if (gated and packed_rows is not None) else n_out
        return PartialSums(ws, ws.take(splits * n * rows), splits)
    return splits


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
            epilogue: int = EPI_STORE, force_splits: int = 0, packed_rows: Optional[int] = None, act: Optional[int] = None) -> int:
    """bfloat16 product on tcgen05.  EPI_STORE: out[t][r] = act(x.w + bias); EPI_ADD: float32 out += x.w + bias;
    EPI_GATED: w from ``pack_weight(w, halves=2)``, out[t][f] = act(x.w_gate[f]) * (x.w_up[f]) (act defaults to SiLU).
    Returns the number of K splits used."""
    if act is None:
        act = ACT_SILU if epilogue == EPI_GATED else ACT_NONE
    return _gemm_tc(x, w, out, bias, epilogue, act, force_splits, False, packed_rows)


def gemm_tc_deferred(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
                     epilogue: int = EPI_STORE, force_splits: int = 0, packed_rows: Optional[int] = None) -> Optional[PartialSums]:
    """The same product, its sum left to the caller when it was cut along K: returns ``PartialSums`` ([splits][n][n_out]
    float32 in a slab of the workspace; `out` is NOT written, and the bias not added) for the caller's next kernel
    (``finish_*``) to sum, then ``release()``.  Returns None when the product was not cut: `out` is complete."""
    r = _gemm_tc(x, w, out, bias, epilogue, ACT_NONE, force_splits, True, packed_rows)
    return r if isinstance(r, PartialSums) else None


def finish_add_rmsnorm(partial: torch.Tensor, splits: int, bias: Optional[torch.Tensor], x: torch.Tensor,
                       w: torch.Tensor, out: torch.Tensor, eps: float) -> None:
    """x += sum of the split-K partials (+ bias); out = RMSNorm(x) * w.  One pass over each row."""
    _dev(x, w, out, bias)
    n, d = x.shape
    assert x.dtype == torch.float32 and w.dtype == torch.float32 and out.shape == (n, d) and partial.numel() >= splits * n * d
    _check(lib().xr_finish_add_rmsnorm(partial.data_ptr(), splits, _ptr(bias), x.data_ptr(), w.data_ptr(), out.data_ptr(),
                                       dtype_code(out.dtype), n, d, float(eps), _stream()), "finish_add_rmsnorm")
    _count()


def finish_plain(partial: torch.Tensor, splits: int, bias: Optional[torch.Tensor], out: torch.Tensor,
                 accumulate: bool) -> None:
    """out (+)= sum of the split-K partials (+ bias)."""
    n, width = out.shape
    assert out.stride(1) == 1 and partial.numel() >= splits * n * width
    _check(lib().xr_finish_plain(partial.data_ptr(), splits, _ptr(bias), out.data_ptr(), dtype_code(out.dtype),
                                 int(accumulate), n, width, out.stride(0), _stream()), "finish_plain")
    _count()


def finish_rope_store(partial: torch.Tensor, splits: int, bias: Optional[torch.Tensor], qkv: torch.Tensor, positions,
                      tok_seg, block_tables, inv_freq: Optional[torch.Tensor], cache_k_ptr: Optional[int],
                      page_stride: int, v_offset: int, H: int, K: int, hd: int, rotary_dim: int, max_pages: int,
                      page_size: int, adjacent: bool = False, mscale: float = 1.0) -> None:
    """Sum the partials of the fused QKV product (+ bias), rotate Q and K, write Q into `qkv` and K, V into
    their pages (into `qkv` when cache_k_ptr is None)."""
    _dev(qkv, positions, tok_seg, block_tables, inv_freq, bias)
    n = qkv.shape[0]
    assert qkv.dtype == torch.bfloat16 and qkv.shape[1] == (H + 2 * K) * hd and partial.numel() >= splits * n * qkv.shape[1]
    _check(lib().xr_finish_rope_store(partial.data_ptr(), splits, _ptr(bias), qkv.data_ptr(), positions.data_ptr(),
                                      tok_seg.data_ptr(), block_tables.data_ptr(), _ptr(inv_freq), cache_k_ptr, page_stride,
                                      v_offset, n, H, K, hd, rotary_dim, max_pages, page_size, int(adjacent), float(mscale),
                                      _stream()), "finish_rope_store")
    _count()


# ---------------------------------------------------------------------------
def attention_mma_supported(dtype: torch.dtype, H: int, K: int, hd: int) -> bool:
    return dtype == torch.bfloat16 and hd % 16 == 0 and 16 <= hd <= 128 and H % K == 0 and H // K <= 16


def attention_mma_splits(max_kv_len: int, window: int, items: int) -> int:
    """Slots of scratch per (segment, kv head) pair that the key-split kernel needs for a step with `items` such
    pairs: its spans per request, or its CTAs over the pairs where it cuts the step's tiles into even shares."""
    return int(lib().xr_attention_mma_splits(max_kv_len, window, items))


def long_row_tiles(seg_len_host, heads_per_kv_head: int, rows_per_tile: int) -> int:
    """Row tiles of the portions that the prompt attention kernels take (more than 16 packed rows = tokens x query heads
    per kv head), summed: the x extent of their grids.  seg_len_host: the portions' lengths (numpy, on the host)."""
    rows = seg_len_host.astype("int64") * heads_per_kv_head
    return int(((rows + rows_per_tile - 1) // rows_per_tile)[rows > 16].sum())


def attention_even_launches() -> int:
    """How often the decode attention was launched in even shares (rather than in spans) so far."""
    return int(lib().xr_attention_even_launches())


def attention_wait_probe(device: torch.device, limit: int = 1 << 12) -> None:
    """Run the decode attention's bounded wait on a flag that nothing raises: it runs out after `limit` looks and the
    status word of `device` says so, as it would for a hand-over that never came (``tc_check_status`` then raises).
    Nothing faults and nothing hangs; this exists so that tests can drive the host's handling of that word."""
    ws = workspace(device)
    _check(lib().xr_attention_wait_probe(ws.flags.data_ptr() + 4 * (ws.flags.numel() - 1), ws.status.data_ptr(), int(limit),
                                         _stream()), "attention_wait_probe")


def attention_mma(q: torch.Tensor, q_row_stride: int, out: torch.Tensor, cache_k_ptr: int, seg_start, seg_len, seg_pos0,
                  block_tables, part_acc: Optional[torch.Tensor], part_ml: Optional[torch.Tensor], page_stride: int,
                  v_offset: int, H: int, K: int, hd: int, max_pages: int, page_size: int, window: int, scale: float,
                  n_seg: int, max_seg_len: int, max_kv_len: int, splits: int, any_short: bool, any_long: bool,
                  group: Optional[tuple] = None, uneven: bool = False, row_tiles: int = 0) -> None:
    """Causal attention over the pages on tensor cores (bfloat16).  Portions with at most 16 packed rows
    (tokens x heads per kv head) go through the key-split kernel and need `part_acc` [n_seg*K*splits*16*hd]
    and `part_ml` [n_seg*K*splits*32] float32 scratch; longer portions through the row-tiled kernel.
    `group` = (pointer to the cache group's array, its pages, its layers, this layer's index) lets the
    key-split kernel fetch whole page blocks with bulk copies (head sizes 64 and 128, power-of-two pages).
    `uneven`: the requests' lengths differ much; the kernel then cuts the tiles of all requests into even shares from
    fewer requests on than it does otherwise.  row_tiles: ``long_row_tiles(lengths, H // K, 64)``, which sizes the
    row-tiled kernel's grid exactly; 0: every portion gets the blocks of the longest."""
    _dev(out, seg_start, seg_len, seg_pos0, block_tables, part_acc, part_ml)
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and out.shape[1] == H * hd
    if any_short:
        assert part_acc is not None and part_acc.numel() >= n_seg * K * splits * 16 * hd
        assert part_ml is not None and part_ml.numel() >= n_seg * K * splits * 32
    ws = workspace(out.device)
    _check(lib().xr_attention_mma(q.data_ptr(), out.data_ptr(), cache_k_ptr, seg_start.data_ptr(), seg_len.data_ptr(),
                                  seg_pos0.data_ptr(), block_tables.data_ptr(), _ptr(part_acc), _ptr(part_ml),
                                  q_row_stride, page_stride, v_offset, n_seg, H, K, hd, max_pages, page_size, window,
                                  float(scale), max_seg_len, max_kv_len, splits, int(any_short), int(any_long),
                                  group[0] if group else None, group[1] if group else 0, group[2] if group else 1,
                                  group[3] if group else 0, ws.status.data_ptr() if group else None,
                                  ws.flags.data_ptr() if group else None, ws.flags.numel() if group else 0, int(uneven),
                                  row_tiles, _stream()), "attention_mma")
    _count((1 if any_long else 0) + (2 if any_short else 0))


def attention_tc_supported(dtype: torch.dtype, H: int, K: int, hd: int, page_size: int) -> bool:
    return dtype == torch.bfloat16 and bool(lib().xr_attention_tc_supported(H, K, hd, page_size))


def attention_tc(qkv: torch.Tensor, out: torch.Tensor, seg_start, seg_len, seg_pos0, block_tables, group: tuple,
                 H: int, K: int, hd: int, max_pages: int, page_size: int, window: int, scale: float, n_seg: int,
                 max_seg_len: int, row_tiles: int = 0) -> None:
    """Causal attention of the portions with more than 16 packed rows on tcgen05 (S and O in tensor memory).
    qkv: the step's fused rows (Q heads first); group = (pointer to the cache group's array, pages, layers, layer).
    row_tiles: ``long_row_tiles(lengths, H // K, 128)``, which sizes the grid exactly; 0: every portion gets the blocks
    of the longest."""
    _dev(qkv, out, seg_start, seg_len, seg_pos0, block_tables)
    n = qkv.shape[0]
    assert qkv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and out.shape == (n, H * hd)
    status = tc_workspace(out.device)[1]
    _check(lib().xr_attention_tc(qkv.data_ptr(), out.data_ptr(), group[0], seg_start.data_ptr(), seg_len.data_ptr(),
                                 seg_pos0.data_ptr(), block_tables.data_ptr(), status.data_ptr(), qkv.stride(0), n, n_seg,
                                 H, K, hd, max_pages, page_size, window, float(scale), max_seg_len, row_tiles, group[1], group[2],
                                 group[3], _stream()), "attention_tc")
    _count()
