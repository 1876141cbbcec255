"""Run one kernel alone on synthetic data and report its time: for tuning and for profiler captures.

    python -m xyntetik_runner_b200.probe gemm --tokens 8 --rows 14336 --k 4096 --epilogue swiglu
    python -m xyntetik_runner_b200.probe attention --batch 8 --context 8192 [--portion 1]

Times are CUDA-event times of `--iters` launches replayed from one CUDA graph (so that launch gaps do not
count), each launch on a different copy of the weights / a different layer of the cache, with more than an
L2's worth of data between two uses of the same bytes.  `--plain` launches without a graph (what a profiler
should be given).
"""
from __future__ import annotations

import argparse
import math
import sys

import torch

from . import kernels

L2_BYTES = 126 << 20


def _time(run, iters: int, plain: bool) -> float:
    for i in range(3):
        run(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if plain:
        e0.record()
        for i in range(iters):
            run(i)
        e1.record()
    else:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(iters):
                run(i)
        g.replay()
        torch.cuda.synchronize()
        e0.record()
        g.replay()
        e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters          # microseconds per launch


def gemm(a) -> None:
    dev = torch.device("cuda:0")
    epi = {"store": kernels.EPI_STORE, "add": kernels.EPI_ADD, "swiglu": kernels.EPI_SWIGLU}[a.epilogue]
    halves = 2 if epi == kernels.EPI_SWIGLU else 1
    rows = a.rows * halves
    nbytes = rows * a.k * 2
    copies = max(2, math.ceil(3 * L2_BYTES / nbytes))
    ws = [kernels.pack_weight((torch.randn(rows, a.k, device=dev) * 0.02).to(torch.bfloat16), halves) for _ in range(copies)]
    x = torch.randn(a.tokens, a.k, device=dev).to(torch.bfloat16)
    out = torch.zeros(a.tokens, a.rows, dtype=torch.float32 if epi == kernels.EPI_ADD else torch.bfloat16, device=dev)

    def run(i):
        kernels.gemm_tc(x, ws[i % copies], out, None, epi, packed_rows=a.rows, force_splits=a.splits)
    us = _time(run, a.iters, a.plain)
    kernels.tc_check_status(dev)
    print(f"gemm tokens={a.tokens} rows={rows} k={a.k} epilogue={a.epilogue}: {us:.1f} us, "
          f"{nbytes / us / 1e3:.0f} GB/s of weights, {2.0 * a.tokens * rows * a.k / us / 1e6:.1f} TFLOP/s")


def attention(a) -> None:
    dev = torch.device("cuda:0")
    H, K, hd, page, B, ctx, L = a.heads, a.kv_heads, a.head_dim, a.page_size, a.batch, a.context, a.portion
    mp = -(-ctx // page)
    n_pages = B * mp
    layer_bytes = n_pages * 2 * K * page * hd * 2
    layers = max(2, math.ceil(3 * L2_BYTES / layer_bytes))
    cache = torch.randn(n_pages, layers, 2, K, page, hd, device=dev).to(torch.bfloat16)
    bt = torch.arange(n_pages, dtype=torch.int32, device=dev).view(B, mp)
    n = B * L
    qkv = torch.randn(n, (H + 2 * K) * hd, device=dev).to(torch.bfloat16)
    out = torch.empty(n, H * hd, dtype=torch.bfloat16, device=dev)
    starts = torch.arange(0, n, L, dtype=torch.int32, device=dev)
    lens = torch.full((B,), L, dtype=torch.int32, device=dev)
    pos0 = torch.full((B,), ctx - L, dtype=torch.int32, device=dev)
    short = L * (H // K) <= 16
    splits = kernels.attention_mma_splits(ctx, 0, B * K)
    pa = torch.empty(B * K * splits * 16 * hd, device=dev)
    pm = torch.empty(B * K * splits * 32, device=dev)

    def run(i):
        kp = cache.data_ptr() + (i % layers) * cache.stride(1) * 2
        if not short and not a.no_tc and kernels.attention_tc_supported(torch.bfloat16, H, K, hd, page):
            kernels.attention_tc(qkv, out, starts, lens, pos0, bt, (cache.data_ptr(), n_pages, layers, i % layers), H, K, hd, mp, page,
                                 0, 1 / math.sqrt(hd), B, L)
            return
        kernels.attention_mma(qkv, qkv.shape[1], out, kp, starts, lens, pos0, bt, pa, pm, cache.stride(0), cache.stride(2),
                              H, K, hd, mp, page, 0, 1 / math.sqrt(hd), B, L, ctx, splits, short, not short,
                              group=None if a.no_tma else (cache.data_ptr(), n_pages, layers, i % layers))
    us = _time(run, a.iters, a.plain)
    kernels.tc_check_status(dev)
    kv_bytes = B * ctx * K * hd * 2 * 2
    flops = 4.0 * B * H * hd * (L * (ctx - L) + L * (L + 1) / 2)
    print(f"attention batch={B} context={ctx} portion={L} heads={H}/{K} head_dim={hd}: {us:.1f} us, "
          f"{kv_bytes / us / 1e3:.0f} GB/s of keys+values, {flops / us / 1e6:.1f} TFLOP/s")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m xyntetik_runner_b200.probe")
    sub = ap.add_subparsers(dest="what", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--tokens", type=int, default=8)
    g.add_argument("--rows", type=int, default=14336, help="output features (per half with --epilogue swiglu)")
    g.add_argument("--k", type=int, default=4096)
    g.add_argument("--epilogue", choices=["store", "add", "swiglu"], default="store")
    g.add_argument("--splits", type=int, default=0, help="force the number of K splits (0: the kernel's own choice)")
    t = sub.add_parser("attention")
    t.add_argument("--batch", type=int, default=8)
    t.add_argument("--context", type=int, default=8192)
    t.add_argument("--portion", type=int, default=1, help="query tokens per request (1: decoding)")
    t.add_argument("--heads", type=int, default=32)
    t.add_argument("--kv-heads", type=int, default=8)
    t.add_argument("--head-dim", type=int, default=128)
    t.add_argument("--page-size", type=int, default=64)
    t.add_argument("--no-tc", action="store_true", help="prompt portions on the mma.sync kernel instead of tcgen05")
    t.add_argument("--no-tma", action="store_true", help="decode kernel with per-thread cp.async gathers instead of bulk copies")
    for p in (g, t):
        p.add_argument("--iters", type=int, default=20)
        p.add_argument("--plain", action="store_true", help="no CUDA graph")
    a = ap.parse_args(argv)
    (gemm if a.what == "gemm" else attention)(a)
    return 0


if __name__ == "__main__":
    sys.exit(main())
