"""Run one kernel alone on synthetic data and report its time: for tuning and for profiler captures.

    python -m xyntetik_runner_b200.probe gemm --tokens 8 --rows 14336 --k 4096 --epilogue swiglu
    python -m xyntetik_runner_b200.probe attention --batch 8 --context 8192 [--portion 1]
    python -m xyntetik_runner_b200.probe sample --rows 8 --vocab 128256 [--one-block]
    XRB200_TRACE=1 python -m xyntetik_runner_b200.probe timeline --batch 8 --context 8192 --layers 8

Times are CUDA-event times of `--iters` launches replayed from one CUDA graph (so that launch gaps do not
count), each launch on a different copy of the weights / a different layer of the cache, with more than an
L2's worth of data between two uses of the same bytes.  `--plain` launches without a graph (what a profiler
should be given).

`timeline` runs decode steps of a random Llama-3-8B-shaped model (a few layers of it) on a library built with
XRB200_TRACE=1, in which the first thread of every launch writes down when it was resident and when the kernel
ahead of it was complete, and prints one layer of one step: for each kernel, how long it took from the moment
it could begin to the moment the next one could.
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


def sample(a) -> None:
    """The sampling kernel on `--rows` rows of random logits, for a few settings of the chain."""
    dev = torch.device("cuda:0")
    rows, V = a.rows, a.vocab
    logits = torch.randn(rows, V, device=dev) * 3
    full = lambda v, dt=torch.float32: torch.full((rows,), v, dtype=dt, device=dev)
    out = torch.zeros(rows, dtype=torch.int32, device=dev)
    scratch = torch.empty(rows * V, dtype=torch.float32, device=dev)
    recent = torch.full((rows, 256), -1, dtype=torch.int32, device=dev)
    recent[:, :40] = torch.randint(0, V, (rows, 40), dtype=torch.int32, device=dev)
    settings = {"greedy": (0.0, 0, 1.0, 0.0, 1.0), "temperature": (0.8, 0, 1.0, 0.0, 1.0), "top-k 40": (0.8, 40, 1.0, 0.0, 1.0),
                "top-k 40, top-p 0.95": (0.8, 40, 0.95, 0.0, 1.0), "top-k 40, top-p 0.95, min-p 0.05, penalty 1.1": (0.8, 40, 0.95, 0.05, 1.1)}
    for name, (temp, k, p, m, pen) in settings.items():
        args = (logits, full(temp), full(k, torch.int32), full(p), full(m), full(pen), full(0.37), recent, scratch, out)
        us = _time(lambda i: kernels.sample(*args, any_sampled=temp > 0, one_block=a.one_block), a.iters, a.plain)
        print(f"sample rows={rows} vocab={V} {name}: {us:.1f} us")


def timeline(a) -> None:
    import ctypes
    import numpy as np
    from .csrc import build
    if not build.TRACE:
        raise SystemExit("the timeline needs the tracing library: run with XRB200_TRACE=1")
    from .config.llama import LlamaConfig
    from .engine.engine import EngineParams, StepEntry, random_engine
    from .sampling.sampler import DeviceSampler, RequestSampler, SamplingParams
    cfg = LlamaConfig.from_dict({
        "architectures": ["LlamaForCausalLM"], "hidden_size": a.hidden, "num_hidden_layers": a.layers, "num_attention_heads": a.heads,
        "num_key_value_heads": a.kv_heads, "head_dim": a.head_dim, "intermediate_size": a.intermediate, "vocab_size": a.vocab, "rms_norm_eps": 1e-5,
        "rope_theta": 500000.0, "max_position_embeddings": a.context, "tie_word_embeddings": False, "hidden_act": "silu",
        "torch_dtype": "bfloat16"})
    B = a.batch
    eng = random_engine(cfg, 2, EngineParams(dtype="bfloat16", max_tokens=B * a.context, page_size=64, max_requests=B,
                                             max_request_tokens=a.context, max_step_tokens=2048))
    for kv in eng.kv:
        kv.normal_(0.0, 1.0)
    sampler = DeviceSampler(eng.device)
    ids = [f"r{i}" for i in range(B)]
    for r in ids:
        eng.adopt(r, a.context - 40)
    samplers = [RequestSampler(SamplingParams()) for _ in ids]
    rng = np.random.RandomState(0)
    lib = kernels.lib()
    lib.xr_trace_dump.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    host = (ctypes.c_ulonglong * (32 * 4096 * 4))()
    counts = (ctypes.c_uint * 32)()
    for s in range(12):
        logits = eng.step([StepEntry(r, [int(rng.randint(0, 1000))], [0]) for r in ids])
        sampler.pick(logits, samplers)
        if s == 10:
            torch.cuda.synchronize()
            lib.xr_trace_dump(host, counts)            # drop what came before the step that is read
    torch.cuda.synchronize()
    n_files = lib.xr_trace_dump(host, counts)
    rec = np.array(host, dtype=np.uint64).reshape(32, 4096, 4)
    ev = []
    for f in range(n_files):
        for k in range(min(int(counts[f]), 4096)):
            t0, t1, g, b = (int(x) for x in rec[f, k])
            ev.append((t1, t0, (g >> 40, (g >> 20) & 0xfffff, g & 0xfffff), b))
    ev.sort()
    # the step that was recorded: embedding, first norm, the same kernels layer after layer (the last finish of the
    # last layer also does the final norm), then head product and sampling; print the second layer and the start
    # of the third
    per_layer = (len(ev) - 4) // a.layers
    if per_layer < 1 or 2 + per_layer * a.layers + 2 != len(ev):
        raise SystemExit(f"{len(ev)} launches were recorded: not embedding + norm + {a.layers} equal layers + 2")
    first = 2 + per_layer
    rows = ev[first:first + per_layer + 1]
    if len(rows) < per_layer + 1:
        raise SystemExit(f"only {len(ev)} launches were recorded")
    print(f"one layer of a decode step, batch {B}, context {a.context} (times in us)")
    print(f"{'could begin':>12} {'resident before':>16} {'took':>7}  grid / block")
    base = rows[0][0]
    for (t1, t0, g, b), nxt in zip(rows[:-1], rows[1:]):
        print(f"{(t1 - base) / 1e3:12.2f} {(t1 - t0) / 1e3:16.2f} {(nxt[0] - t1) / 1e3:7.2f}  {g} / {b}")
    print(f"layer: {(rows[-1][0] - base) / 1e3:.2f} us")
    # the two ends of the last recorded step: embedding and first norm; last finish + final norm, head, sampling
    step = ev
    print("start and end of the step:")
    for idx in (0, 1, len(step) - 3, len(step) - 2):
        (t1, t0, g, b), nxt = step[idx], step[idx + 1]
        print(f"{(t1 - step[0][0]) / 1e3:12.2f} {(t1 - t0) / 1e3:16.2f} {(nxt[0] - t1) / 1e3:7.2f}  {g} / {b}")
    print(f"step up to the sampling kernel: {(step[-1][0] - step[0][0]) / 1e3:.2f} us")


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
    sm = sub.add_parser("sample")
    sm.add_argument("--rows", type=int, default=8)
    sm.add_argument("--vocab", type=int, default=128256)
    sm.add_argument("--one-block", action="store_true", help="one block a row whatever the width (no cluster)")
    tl = sub.add_parser("timeline")
    tl.add_argument("--batch", type=int, default=8)
    tl.add_argument("--context", type=int, default=8192)
    tl.add_argument("--layers", type=int, default=8)
    tl.add_argument("--hidden", type=int, default=4096)
    tl.add_argument("--heads", type=int, default=32)
    tl.add_argument("--kv-heads", type=int, default=8)
    tl.add_argument("--head-dim", type=int, default=128)
    tl.add_argument("--intermediate", type=int, default=14336)
    tl.add_argument("--vocab", type=int, default=128256)
    for p in (g, t, sm):
        p.add_argument("--iters", type=int, default=20)
        p.add_argument("--plain", action="store_true", help="no CUDA graph")
    a = ap.parse_args(argv)
    {"gemm": gemm, "attention": attention, "sample": sample, "timeline": timeline}[a.what](a)
    return 0


if __name__ == "__main__":
    sys.exit(main())
