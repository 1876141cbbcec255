"""Per-kernel times of a model shape: each dominant kernel of a step alone, on data larger than L2.

``kernel_table(config, tokens, context, ...)`` times the products (QKV, O, gate/up with SwiGLU, down, head), the
attention and the sampling kernel at the sizes of `config`, for a step of `tokens` single-token requests at `context`
(decode) or one prompt portion of `tokens` tokens, and returns rows
``{"kernel", "us", "bytes" | "flop", "rate", "unit", "peak", "frac"}``: bytes are what the kernel must read once
(weights; keys and values), FLOP what it must compute, `frac` the achieved rate over the measured peak for its
bound.  Times are CUDA-event times of launches replayed from one CUDA graph (launch gaps do not count), every launch
on another copy of its weights or another layer of the cache, with more than an L2's worth of bytes between two uses
of the same data.  Used by ``bench.py --kernels`` and by ``runner --bench-json`` (the reference's --bench-json reports
only the two phase rates, src/main.c:1435-1515).
"""
from __future__ import annotations

import json
import math
import os
from typing import Callable, Dict, List, Optional

import torch

from . import kernels

L2_BYTES = 126 << 20
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks(root: Optional[str] = None) -> Dict[str, object]:
    """Measured copy bandwidth and bfloat16 product rate of this pool's GPUs (MEASURED_PEAKS.json beside the
    package's parent folder, written by whoever measured them), else an earlier measurement as a fallback."""
    root = root or os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    out: Dict[str, object] = dict(FALLBACK_PEAKS, source="fallback")
    try:
        with open(p) as f:
            d = json.load(f)
        for k in FALLBACK_PEAKS:
            if isinstance(d.get(k), (int, float)) and d[k] > 0:
                out[k] = float(d[k])
        out["source"] = "measured"
    except (OSError, ValueError):
        pass
    return out


def time_replayed(run: Callable[[int], None], iters: int = 20, plain: bool = False) -> float:
    """Microseconds per call of run(i), i = 0..iters-1, replayed from one CUDA graph (or launched one by one)."""
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
    return e0.elapsed_time(e1) * 1e3 / iters


def time_product(tokens: int, rows: int, k: int, epilogue: str, iters: int = 20, plain: bool = False, splits: int = 0,
                 device: str = "cuda:0") -> float:
    """One tensor-core product [tokens, k] x [rows, k]^T (rows per half for "swiglu") on packed weights, with its
    split-K finish when it is split."""
    dev = torch.device(device)
    epi = {"store": kernels.EPI_STORE, "add": kernels.EPI_ADD, "swiglu": kernels.EPI_SWIGLU, "logits": kernels.EPI_STORE}[epilogue]
    halves = 2 if epi == kernels.EPI_SWIGLU else 1
    nbytes = rows * halves * k * 2
    copies = max(2, math.ceil(3 * L2_BYTES / nbytes))
    ws = []
    for _ in range(copies):
        w = torch.empty(rows * halves, k, dtype=torch.bfloat16, device=dev).normal_(0.0, 0.02)
        ws.append(kernels.pack_weight(w, halves))
        del w
    x = torch.randn(tokens, k, device=dev).to(torch.bfloat16)
    out = torch.zeros(tokens, rows, dtype=torch.float32 if epilogue in ("add", "logits") else torch.bfloat16, device=dev)
    torch.cuda.synchronize()
    us = time_replayed(lambda i: kernels.gemm_tc(x, ws[i % copies], out, None, epi, packed_rows=rows, force_splits=splits),
                       iters, plain)
    kernels.tc_check_status(dev)
    return us


def time_attention(batch: int, context: int, portion: int, heads: int, kv_heads: int, head_dim: int, page_size: int = 64,
                   iters: int = 20, plain: bool = False, use_tc: bool = True, use_tma: bool = True, device: str = "cuda:0",
                   spread: bool = False) -> float:
    """Attention of `batch` requests whose last `portion` tokens are in the step, each at `context` tokens
    (`spread`: at lengths from an eighth of `context` up to `context`, evenly; ``spread_lengths`` gives them)."""
    dev = torch.device(device)
    H, K, hd, page, B, ctx, L = heads, kv_heads, head_dim, page_size, batch, context, portion
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
    if spread:
        pos0 = torch.tensor([c - L for c in spread_lengths(B, ctx, L)], dtype=torch.int32, device=dev)
    short = L * (H // K) <= 16
    splits = kernels.attention_mma_splits(ctx, 0, B * K)
    pa = torch.empty(B * K * splits * 16 * hd, device=dev)
    pm = torch.empty(B * K * splits * 32, device=dev)
    tc = not short and use_tc and kernels.attention_tc_supported(torch.bfloat16, H, K, hd, page)

    def run(i):
        if tc:
            kernels.attention_tc(qkv, out, starts, lens, pos0, bt, (cache.data_ptr(), n_pages, layers, i % layers), H, K, hd, mp, page,
                                 0, 1 / math.sqrt(hd), B, L)
            return
        kp = cache.data_ptr() + (i % layers) * cache.stride(1) * 2
        kernels.attention_mma(qkv, qkv.shape[1], out, kp, starts, lens, pos0, bt, pa, pm, cache.stride(0), cache.stride(2),
                              H, K, hd, mp, page, 0, 1 / math.sqrt(hd), B, L, ctx, splits, short, not short,
                              group=(cache.data_ptr(), n_pages, layers, i % layers) if use_tma else None, uneven=spread)
    us = time_replayed(run, iters, plain)
    kernels.tc_check_status(dev)
    return us


def spread_lengths(batch: int, context: int, portion: int = 1):
    """Lengths from an eighth of `context` up to `context`, evenly (never shorter than the portion)."""
    lo = max(portion, context // 8)
    return [lo + (context - lo) * i // max(1, batch - 1) for i in range(batch)]


def time_sampling(rows: int, vocab: int, setting: str = "greedy", iters: int = 20, plain: bool = False, one_block: bool = False,
                  device: str = "cuda:0", shortcuts: bool = True, flat: bool = False) -> float:
    """Rows of logits shaped like a model's: a body of small values and, in every row, 64 tokens that stand out by
    up to 14 (the best few carry most of the mass).  `flat`: plain normal values of deviation 3, whose mass is spread
    over thousands of tokens, so that without top-k the head of the distribution does not hold what is needed."""
    dev = torch.device(device)
    settings = {"greedy": (0.0, 0, 1.0, 0.0, 1.0), "temperature": (0.8, 0, 1.0, 0.0, 1.0), "top-k 40": (0.8, 40, 1.0, 0.0, 1.0),
                "top-k 40, top-p 0.95": (0.8, 40, 0.95, 0.0, 1.0), "top-k 40, top-p 0.95, min-p 0.05, penalty 1.1": (0.8, 40, 0.95, 0.05, 1.1)}
    temp, k, p, m, pen = settings[setting]
    if flat:
        logits = torch.randn(rows, vocab, device=dev) * 3
    else:
        logits = torch.randn(rows, vocab, device=dev) * 1.5
        lift = 14.0 - 0.2 * torch.arange(64, device=dev, dtype=torch.float32)
        for r in range(rows):
            logits[r, torch.randperm(vocab, device=dev)[:64]] += lift
    full = lambda v, dt=torch.float32: torch.full((rows,), v, dtype=dt, device=dev)
    out = torch.zeros(rows, dtype=torch.int32, device=dev)
    scratch = torch.empty(rows * vocab, dtype=torch.float32, device=dev)
    recent = torch.full((rows, 256), -1, dtype=torch.int32, device=dev)
    recent[:, :40] = torch.randint(0, vocab, (rows, 40), dtype=torch.int32, device=dev)
    args = (logits, full(temp), full(k, torch.int32), full(p), full(m), full(pen), full(0.37), recent, scratch, out)
    return time_replayed(lambda i: kernels.sample(*args, any_sampled=temp > 0, one_block=one_block, shortcuts=shortcuts), iters, plain)


SAMPLING_SETTINGS = ("greedy", "temperature", "top-k 40", "top-k 40, top-p 0.95", "top-k 40, top-p 0.95, min-p 0.05, penalty 1.1")


def kernel_table(cfg, tokens: int, context: int, decode: bool = True, pk: Optional[Dict[str, object]] = None,
                 iters: int = 20, device: str = "cuda:0") -> List[Dict[str, object]]:
    """Rows for the dominant kernels of one step at the sizes of `cfg` (any configuration with Llama's size
    fields).  decode: `tokens` requests of one token each at `context`; else one portion of `tokens` tokens ending
    at `context`."""
    pk = pk or peaks()
    d, H, K, hd, F, V = cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.intermediate_size, cfg.vocab_size
    rows: List[Dict[str, object]] = []
    head_rows = tokens if decode else 1

    def add(name, us, nbytes, flop):
        hbm, tf = float(pk["hbm_gbs"]), float(pk["bf16_tflops"])
        by_bytes = nbytes / us / 1e3              # GB/s
        by_flop = flop / us / 1e6                 # TFLOP/s
        if by_bytes / hbm >= by_flop / tf:
            rows.append({"kernel": name, "us": round(us, 2), "bytes": int(nbytes), "rate": round(by_bytes, 1), "unit": "GB/s",
                         "peak": hbm, "frac": round(by_bytes / hbm, 3)})
        else:
            rows.append({"kernel": name, "us": round(us, 2), "flop": float(flop), "rate": round(by_flop, 1), "unit": "TFLOP/s",
                         "peak": tf, "frac": round(by_flop / tf, 3)})
    for name, n_out, k, epi, tk in (("qkv product", (H + 2 * K) * hd, d, "store", tokens), ("o product + residual", d, H * hd, "add", tokens),
                                    ("gate/up product + SwiGLU", F, d, "swiglu", tokens), ("down product + residual", d, F, "add", tokens),
                                    ("head product", V, d, "logits", head_rows)):
        halves = 2 if epi == "swiglu" else 1
        us = time_product(tk, n_out, k, epi, iters=iters, device=device)
        add(f"{name} [{tk} x {k}] x [{n_out * halves} x {k}]", us, n_out * halves * k * 2, 2.0 * tk * n_out * halves * k)
        torch.cuda.empty_cache()
    if decode:
        us = time_attention(tokens, context, 1, H, K, hd, iters=iters, device=device)
        add(f"attention, {tokens} requests x 1 token at {context}", us, tokens * context * K * hd * 2 * 2, 4.0 * tokens * H * hd * context)
    else:
        us = time_attention(1, context, tokens, H, K, hd, iters=iters, device=device)
        add(f"attention, portion of {tokens} ending at {context}", us, context * K * hd * 2 * 2,
            4.0 * H * hd * (tokens * (context - tokens) + tokens * (tokens + 1) / 2))
    torch.cuda.empty_cache()
    us = time_sampling(head_rows, V, "greedy", iters=iters, device=device)
    add(f"sampling (argmax), {head_rows} rows of {V}", us, head_rows * V * 4, 0.0)
    return rows
