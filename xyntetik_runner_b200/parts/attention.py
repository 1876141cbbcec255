"""Grouped-query causal attention over the paged cache.

q = Wq h (+bq), k = Wk h (+bk), v = Wv h (+bv) as one fused product; Q and K are
rotated by the position encoding after the projection and before the cache
write, V is stored as it is (src/model.c:6243-6310).  Query head h reads kv
head h / (H/K); scores are (q . k) * scale over the keys t0..p, softmax in
float32, weighted sum of V (src/model.c:3548-3589); then x += Wo o (+bo)
(src/model.c:6338, 6350-6352).  Heads, kv heads, head size, scale, window and
position encoding are all arguments.
"""
from __future__ import annotations

import math
import os
from typing import Optional

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import KVNeed, Mixer, PositionEncoding, register_mixer
from .linear import Linear

# Which attention kernels the mixer may use (module attributes, so that a test can compare paths): the mma.sync kernels
# for bfloat16 (else the float32-arithmetic kernel), the tcgen05 kernel for prompt portions, bulk copies in the decode
# kernel.  XRB200_NO_TMA_ATTENTION=1 (read once) keeps the decode kernel on per-thread cp.async gathers: a test runs
# generation both ways in child processes and compares the tokens.
USE_MMA = True
USE_TC = True
USE_TMA = os.environ.get("XRB200_NO_TMA_ATTENTION", "0") in ("", "0")
counters = {"mma": 0, "simt": 0, "tcgen05": 0}


class GQAAttention(Mixer):
    graph_safe = True
    def __init__(self, width: int, heads: int, kv_heads: int, head_dim: int, position: PositionEncoding,
                 prefix: str, bias: bool = False, window: Optional[int] = None, scale: Optional[float] = None,
                 q: str = "q_proj", k: str = "k_proj", v: str = "v_proj", o: str = "o_proj"):
        if heads % kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        if not (1 <= head_dim <= 256):
            raise ValueError(f"head_dim {head_dim}: the attention kernels take head sizes up to 256")
        self.width, self.H, self.K, self.hd = width, heads, kv_heads, head_dim
        self.position, self.prefix, self.bias, self.window = position, prefix, bias, window
        self.scale = 1.0 / math.sqrt(head_dim) if scale is None else float(scale)   # src/model.h:464-467
        self.proj = (q, k, v, o)
        self.qkv = self.out = None
        self.rot = None

    def kv_need(self):
        return KVNeed(self.K, self.hd, self.window)

    def tensors(self):
        q, k, v, o = (self.prefix + n for n in self.proj)
        qd, kd = self.H * self.hd, self.K * self.hd
        t = {q + ".weight": TensorSpec((qd, self.width)), k + ".weight": TensorSpec((kd, self.width)),
             v + ".weight": TensorSpec((kd, self.width)), o + ".weight": TensorSpec((self.width, qd))}
        if self.bias:
            t.update({q + ".bias": TensorSpec((qd,), "vector", "zeros"), k + ".bias": TensorSpec((kd,), "vector", "zeros"),
                      v + ".bias": TensorSpec((kd,), "vector", "zeros"), o + ".bias": TensorSpec((self.width,), "vector", "zeros")})
        return t

    def bind(self, tensors, rt):
        q, k, v, o = (self.prefix + n for n in self.proj)
        ws = [tensors.pop(n + ".weight") for n in (q, k, v)]
        if len({w.dtype for w in ws}) > 1:
            ws = [w.to(torch.float32) for w in ws]
        bias = obias = None
        if self.bias:
            bias = torch.cat([tensors[n + ".bias"].to(torch.float32) for n in (q, k, v)])
            obias = tensors[o + ".bias"]
        self.qkv = Linear(torch.cat(ws, dim=0), bias).prepare(rt)
        del ws
        self.out = Linear(tensors[o + ".weight"], obias).prepare(rt)
        self.position.prepare(rt)
        try:
            rot = self.position.rotary()
        except NotImplementedError as e:
            raise ValueError(f"{self.prefix}: this mixer takes position encodings that rotate query and key pairs, or "
                             f"none ({e}); another kind needs a mixer of its own") from None
        if rot is not None and rot.rotary_dim > self.hd:
            raise ValueError(f"{self.prefix}: rotary_dim {rot.rotary_dim} exceeds head_dim {self.hd}")
        # (rotary_dim, inv_freq, adjacent pairs, mscale) as the rotation kernels take them
        self.rot = (0, None, False, 1.0) if rot is None or rot.rotary_dim == 0 else \
            (rot.rotary_dim, rot.inv_freq, rot.pairing == "adjacent", rot.mscale)

    def weight_bytes(self):
        return self.qkv.nbytes() + self.out.nbytes()

    @staticmethod
    def _portions(ctx, G):
        """(some portion has at most 16 packed rows, some has more, the longest portion, the row tiles of the longer
        ones in tiles of 128 and of 64 rows)"""
        seg_len = ctx.host["seg_len"]
        rows = seg_len * G
        return (bool((rows <= 16).any()), bool((rows > 16).any()), int(seg_len.max()),
                kernels.long_row_tiles(seg_len, G, 128), kernels.long_row_tiles(seg_len, G, 64))

    def forward(self, ctx, h, x, lay):
        n = h.shape[0]
        qkv_dim = (self.H + 2 * self.K) * self.hd
        qkv = ctx.buf("attn_qkv", (n, qkv_dim), ctx.act_dtype)
        pend = self.qkv.forward(h, qkv, defer=True)
        k_ptr, page_stride, v_offset = ctx.cache_layer(lay)
        bt = ctx.block_tables[lay.group]
        store_ptr = k_ptr if lay.writes_cache else None
        rot_dim, rot_freq, adjacent, mscale = self.rot
        if pend is not None and lay.writes_cache:
            # the product was split along K: its finish, the rotation and the page store are one kernel
            kernels.finish_rope_store(pend.partial, pend.splits, pend.bias, qkv, ctx.positions, ctx.tok_seg, bt,
                                      rot_freq, store_ptr, page_stride, v_offset, self.H, self.K, self.hd,
                                      rot_dim, ctx.max_pages, ctx.page_size, adjacent, mscale)
            pend.release()
        else:
            if pend is not None:
                pend.finish()
            kernels.rope_store(qkv, ctx.positions, ctx.tok_seg, bt, rot_freq, store_ptr, page_stride,
                               v_offset, self.H, self.K, self.hd, rot_dim, ctx.max_pages, ctx.page_size, adjacent, mscale)
        o = ctx.buf("attn_out", (n, self.H * self.hd), ctx.act_dtype)
        # Q is read in place from the fused rows (row stride = qkv_dim)
        G = self.H // self.K
        if USE_MMA and kernels.attention_mma_supported(ctx.act_dtype, self.H, self.K, self.hd):
            # (what the portions' lengths say is the same for every layer of the step)
            any_short, any_long, longest, tiles_tc, tiles_rows = ctx.once(("gqa_portions", G), lambda: self._portions(ctx, G))
            splits = ctx.once(("gqa_splits", self.window or 0, self.K),
                              lambda: kernels.attention_mma_splits(ctx.max_kv_len, self.window or 0, ctx.n_seg * self.K))
            pa = pm = None
            if any_short:
                pa = ctx.buf("attn_part_acc", (ctx.n_seg * self.K * splits * 16 * self.hd,), torch.float32)
                pm = ctx.buf("attn_part_ml", (ctx.n_seg * self.K * splits * 32,), torch.float32)
            if any_long and USE_TC and kernels.attention_tc_supported(ctx.act_dtype, self.H, self.K, self.hd, ctx.page_size):
                # prompt portions: S = Q K^T and O += P V on tcgen05
                kernels.attention_tc(qkv, o, ctx.seg_start, ctx.seg_len, ctx.seg_pos0, bt, ctx.cache_group(lay), self.H,
                                     self.K, self.hd, ctx.max_pages, ctx.page_size, self.window or 0, self.scale, ctx.n_seg,
                                     longest, row_tiles=tiles_tc)
                counters["tcgen05"] += 1
                any_long = False
            if any_short or any_long:
                kernels.attention_mma(qkv, qkv_dim, o, k_ptr, ctx.seg_start, ctx.seg_len, ctx.seg_pos0, bt, pa, pm,
                                      page_stride, v_offset, self.H, self.K, self.hd, ctx.max_pages, ctx.page_size,
                                      self.window or 0, self.scale, ctx.n_seg, longest, ctx.max_kv_len, splits,
                                      any_short, any_long, group=ctx.cache_group(lay) if USE_TMA else None, uneven=ctx.uneven,
                                      row_tiles=tiles_rows)
                counters["mma"] += 1
        else:
            kernels.attention_simt(qkv, qkv_dim, o, k_ptr, ctx.positions, ctx.tok_seg, bt, page_stride, v_offset,
                                   self.H, self.K, self.hd, ctx.max_pages, ctx.page_size, self.window or 0, self.scale)
            counters["simt"] += 1
        ctx.set_pending(x, self.out.forward(o, x, accumulate=True, defer=True))


register_mixer("gqa_attention", GQAAttention)
