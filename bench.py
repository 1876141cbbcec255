#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Llama-3-8B shape, random weights, one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--regions R] [--layers L]
    python bench.py --impl reference                        # the unmodified reference program on the same shape (baseline/reference_arm.py)
    python bench.py --shape llama-2-13b --context 3840      # the same measurement at another shape of the architecture
    python bench.py --workload mixed                        # 64 requests of 16..4,096 tokens through Runner.generate
    python bench.py --kernels [--batch B] [--context C]     # only the per-kernel table (each dominant kernel alone)
    python bench.py --kernel gemm --tokens 8 --rows 4096 --k 14336 --epilogue add [--plain]     # one kernel alone (for a profiler)
    XRB200_TRACE=1 python bench.py --timeline --batch 8 --layers 8                              # one layer of a decode step, kernel by kernel

A "step" is one decode step of the whole batch through the engine's step function and the device sampler.  One JSON
line is printed:
  value     decoded tokens per second at batch 8 with every request at the benchmark context: the median of R regions
            of exactly K steps each, timed on the device with CUDA events (min and max beside it);
  e2e       the same rate through the Python entry point alone (Runner.generate on real prompts of context length,
            host token ids in, sampled ids back on the host every step), over K steps while all requests decode;
  prefill   a 2,048-token prompt in one step; frac = its FLOPs / its time / the measured bfloat16 product peak;
  roofline  bytes the decode step must read (every weight once + the live requests' keys and values) / its time /
            the measured copy bandwidth;
  points    decode at batch 1 and 64 at the benchmark context, and at batch 1/8/64 around context 640 (the
            512-token prompt + 256 generated workload), each with its ms, bytes and fraction; e2e_points: that
            workload through Runner.generate (prompt tok/s and decode tok/s);
  kernels   each dominant kernel of the decode step and of the prefill step alone (xyntetik_runner_b200/measure.py).
This program measures one GPU only.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA3_8B = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "num_hidden_layers": 32, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336, "vocab_size": 128256,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "rope_scaling": None, "max_position_embeddings": 8192,
    "tie_word_embeddings": False, "hidden_act": "silu", "torch_dtype": "bfloat16",
}
LLAMA32_1B = dict(LLAMA3_8B, hidden_size=2048, num_hidden_layers=16, head_dim=64, intermediate_size=8192, tie_word_embeddings=True,
                  rope_scaling={"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                "original_max_position_embeddings": 8192})
LLAMA2_13B = dict(LLAMA3_8B, hidden_size=5120, num_hidden_layers=40, num_attention_heads=40, num_key_value_heads=40,
                  intermediate_size=13824, vocab_size=32000, rope_theta=10000.0, max_position_embeddings=4096)
# shape name -> (config.json keys, weight seed, default context of the decode measurement, name in the metric)
SHAPES = {"llama-3-8b": (LLAMA3_8B, 2, 8192, "Llama-3-8B"), "llama-3.2-1b": (LLAMA32_1B, 3, 8192, "Llama-3.2-1B"),
          "llama-2-13b": (LLAMA2_13B, 4, 3840, "Llama-2-13B")}
FULL_LAYERS = 32
CONTEXT = 8192


class ClockSampler:
    """nvidia-smi sampling of SM clocks and throttle reasons while the timed regions run."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def shape_config(args):
    """(typed configuration, seed, context, shape name, layers of the full model) from --shape / --layers / --context."""
    from xyntetik_runner_b200.config.llama import LlamaConfig
    shape = args.shape or "llama-3-8b"
    shape_cfg, seed, shape_ctx, shape_name = SHAPES[shape]
    full_layers = shape_cfg["num_hidden_layers"]
    layers = args.layers if (args.shape is None or args.layers != FULL_LAYERS) else full_layers
    ctx = args.context if (args.shape is None or args.context != CONTEXT) else shape_ctx
    cfgd = dict(shape_cfg, num_hidden_layers=layers, max_position_embeddings=max(shape_cfg["max_position_embeddings"], ctx))
    return LlamaConfig.from_dict(cfgd), cfgd, seed, ctx, shape, shape_name, full_layers


def reference_arm(args) -> int:
    """The reference's own program on the same layer sizes and weights law: its stock --bench-json (one sequence:
    its command line has no batch), 512-token prompt, 256 tokens decoded."""
    from baseline import reference_arm as ra
    cfg, cfgd, seed, ctx, shape, shape_name, full_layers = shape_config(args)
    n_new = 256
    clocks = ClockSampler()
    clocks.start()
    try:
        out = ra.run(cfgd, seed, n_new, ctx)
    except Exception as e:                       # noqa: BLE001 -- whatever went wrong, the arm answers with one line
        out = {"unavailable": " ".join(f"{type(e).__name__}: {e}".split())[:300]}
    clk = clocks.stop()
    if "unavailable" in out:
        print(json.dumps({"impl": "reference", "unavailable": out["unavailable"]}))
        return 0
    line = {
        "impl": "reference",
        "metric": f"decode tok/s at batch 1 ({shape_name} shape, bf16 weights, 512-token prompt, {n_new} generated): the reference's "
                  "command line runs one sequence; compare with points.decode_b1_ctx640 and e2e_points.b1 of this repository's line",
        "value": out["gen_tok_s"], "unit": "tok/s", "n_gpus": 1, "steps": int(out["generated_tokens"]), "warmup": 0,
        "ms_per_step": 1e3 / out["gen_tok_s"] if out["gen_tok_s"] > 0 else None, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 weights, f32 activations, f16 keys/values (the reference's GPU path)",
        "data": f"synthetic (random weights seed {seed}, the reference's own filler prompt)",
        "config": {"model": shape + "-shape", "layers": cfg.num_hidden_layers, "layers_of_model": full_layers, "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "global_batch": 1, "seq_len": 512 + n_new,
                   "context_allocated": ctx, "parallelism": "single-gpu"},
        "prefill": {"value": out["prompt_tok_s"], "tokens": int(out["prompt_tokens"]), "ms": out["prompt_s"] * 1e3},
        "e2e": {"value": out["gen_tok_s"], "unit": "tok/s", "note": "the reference's timing is wall clock around its own loop, host in the loop"},
        "command": "baseline/_ref/runner -m <file>.gguf --bench-json -n 256 -c %d --gpu auto" % ctx,
        "reference_json": {k: out[k] for k in ("arch", "context", "gpu_layers", "layers", "prompt_tokens", "generated_tokens",
                                                "prompt_tok_s", "gen_tok_s", "prompt_s", "gen_s") if k in out},
        "how": out.get("how"), "model_file_gb": out.get("file_gb"), "clocks": clk,
    }
    print(json.dumps(line))
    return 0


def mixed_workload(args) -> int:
    """64 requests at once with prompts of 16 to 4,096 random tokens (uniform), 128 tokens generated for each, through
    the Python entry point: prompt portions share steps with decoded tokens under the scheduler's token budget.
    Wall-clock time of the second of two runs (the first warms up graphs and buffers); host token ids in and out."""
    import numpy as np
    import torch
    from xyntetik_runner_b200 import kernels
    from xyntetik_runner_b200.config.llama import LlamaConfig
    from xyntetik_runner_b200.engine.runner import Runner
    shape = args.shape or "llama-3.2-1b"
    cfgd, seed, _, _ = SHAPES[shape]
    cfg = LlamaConfig.from_dict(cfgd)
    n_req, new = 64, 128
    rng = np.random.RandomState(seed)
    lens = rng.randint(16, 4097, size=n_req)
    prompts = [[int(t) for t in rng.randint(0, cfg.vocab_size, size=int(n))] for n in lens]
    runner = Runner(config=cfg, random_seed=seed, ctx=4096 + new + 32, batch=2048, parallel=n_req)
    clocks = ClockSampler()
    clocks.start()
    out = None
    for rep in range(2):
        torch.cuda.synchronize()
        launches0, t0 = kernels.launch_count, time.perf_counter()
        res = runner.generate(prompts, n=new, ignore_eos=True)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        gen = sum(len(r.tokens) for r in res)
        out = {"workload": f"{n_req} requests at once, prompts uniform in [16, 4096], {new} generated each, prompt portions mixed with decoding",
               "model": shape + "-shape", "dtype": "bf16", "data": f"synthetic (random weights seed {seed}, random token ids)",
               "seconds": dt, "prompt_tokens": int(lens.sum()), "generated_tokens": gen,
               "value": (int(lens.sum()) + gen) / dt, "unit": "tok/s (prompt + generated)", "generated_tok_s": gen / dt,
               "steps": runner.scheduler.stats.get("steps"), "gpu_launches": kernels.launch_count - launches0,
               "steps_launched_ahead": runner.scheduler.stats.get("steps_launched_ahead"), "step_token_budget": 2048}
    out["clocks"] = clocks.stop()
    if args.step_log:
        # once more, step by step: what each step held and how long the host waited for it
        sch = runner.scheduler
        for p in prompts:
            runner.submit(p, new, ignore_eos=True)
        torch.cuda.synchronize()
        lines, seen = [], dict(sch.stats)
        while sch.has_work():
            t0 = time.perf_counter()
            res = sch.step()
            ms = (time.perf_counter() - t0) * 1e3
            now = dict(sch.stats)
            lines.append(f"{len(lines)} {'ahead' if now['steps_launched_ahead'] > seen['steps_launched_ahead'] else 'plain'} "
                         f"tokens_out={len(res)} prompt_tokens={now['prefill_tokens'] - seen['prefill_tokens']} "
                         f"decode_tokens={now['decode_tokens'] - seen['decode_tokens']} ms={ms:.2f}")
            seen = now
        sch.finished.clear()
        with open(args.step_log, "w") as f:
            f.write("# step, launched-ahead or plain, tokens returned, prompt tokens run, decoded tokens run, wall ms of Scheduler.step\n")
            f.write("\n".join(lines) + "\n")
    print(json.dumps(out))
    return 0


def one_kernel(args) -> int:
    """One kernel alone on synthetic data, its time and rate: for tuning and for profiler captures (--plain: no graph)."""
    from xyntetik_runner_b200 import measure
    it, plain = args.iters, args.plain
    if args.kernel == "gemm":
        halves = 2 if args.epilogue == "swiglu" else 1
        us = measure.time_product(args.tokens, args.rows, args.k, args.epilogue, it, plain, args.splits)
        nbytes = args.rows * halves * args.k * 2
        print(f"gemm tokens={args.tokens} rows={args.rows * halves} k={args.k} epilogue={args.epilogue}: {us:.1f} us, "
              f"{nbytes / us / 1e3:.0f} GB/s of weights, {2.0 * args.tokens * args.rows * halves * args.k / us / 1e6:.1f} TFLOP/s")
    elif args.kernel == "attention":
        B, ctx, L, H, K, hd = args.batch, args.context, args.portion, args.heads, args.kv_heads, args.head_dim
        us = measure.time_attention(B, ctx, L, H, K, hd, args.page_size, it, plain, not args.no_tc, not args.no_tma, spread=args.spread)
        lengths = measure.spread_lengths(B, ctx, L) if args.spread else [ctx] * B
        flops = sum(4.0 * H * hd * (L * (c - L) + L * (L + 1) / 2) for c in lengths)
        print(f"attention batch={B} context={ctx}{' (lengths spread from an eighth of it)' if args.spread else ''} portion={L} heads={H}/{K} head_dim={hd}: {us:.1f} us, "
              f"{sum(lengths) * K * hd * 4 / us / 1e3:.0f} GB/s of keys+values, {flops / us / 1e6:.1f} TFLOP/s")
    else:
        for name in measure.SAMPLING_SETTINGS:
            us = measure.time_sampling(args.sample_rows, args.vocab, name, it, plain, args.one_block, shortcuts=not args.long_way, flat=args.flat)
            print(f"sample rows={args.sample_rows} vocab={args.vocab} {name}: {us:.1f} us")
    return 0


def timeline(args) -> int:
    """One layer of a decode step, kernel by kernel, from a library built with XRB200_TRACE=1 (csrc/build.py): the first
    thread of every launch writes down when it was resident and when the kernel ahead of it was complete."""
    import ctypes
    import numpy as np
    import torch
    from xyntetik_runner_b200 import kernels
    from xyntetik_runner_b200.csrc import build
    if not build.TRACE:
        raise SystemExit("the timeline needs the tracing library: run with XRB200_TRACE=1")
    from xyntetik_runner_b200.engine.engine import EngineParams, StepEntry, random_engine
    from xyntetik_runner_b200.sampling.sampler import DeviceSampler, RequestSampler, SamplingParams
    cfg, _, seed, ctx, _, _, _ = shape_config(args)
    B, n_layers = args.batch, cfg.num_hidden_layers
    mixed = args.mixed and args.portion > 1      # --mixed: a prompt portion of --portion tokens beside --batch decoded tokens
    eng = random_engine(cfg, seed, EngineParams(dtype="bfloat16", max_tokens=(B + (1 if mixed else 0)) * ctx, page_size=64,
                                                max_requests=B + (1 if mixed else 0), max_request_tokens=ctx,
                                                max_step_tokens=max(2048, args.portion + B)))
    for kv in eng.kv:
        kv.normal_(0.0, 1.0)
    sampler = DeviceSampler(eng.device)
    ids = [f"r{i}" for i in range(B)]
    for r in ids:
        eng.adopt(r, ctx - 40)
    samplers = [RequestSampler(SamplingParams()) for _ in ids]
    rng = np.random.RandomState(0)
    lib = kernels.lib()
    lib.xr_trace_dump.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    host = (ctypes.c_ulonglong * (32 * 4096 * 4))()
    counts = (ctypes.c_uint * 32)()
    if args.portion > 1 and not mixed:
        # a prompt step instead: one request of --portion tokens in one step
        for r in ids:
            eng.end(r)
        ids, samplers = ids[:1], samplers[:1]
    for s in range(12):
        if mixed:
            # the portion continues a prompt that already holds half of the context
            eng.adopt("prompt", max(64, ctx // 2 - args.portion))
            logits = eng.step([StepEntry(r, [int(rng.randint(0, 1000))], [0]) for r in ids] +
                              [StepEntry("prompt", [int(t) for t in rng.randint(0, 1000, size=args.portion)], [])])
        elif args.portion > 1:
            logits = eng.step([StepEntry(ids[0], [int(t) for t in rng.randint(0, 1000, size=args.portion)], [args.portion - 1])])
        else:
            logits = eng.step([StepEntry(r, [int(rng.randint(0, 1000))], [0]) for r in ids])
        sampler.pick(logits, samplers)
        if mixed:
            eng.end("prompt")
        elif args.portion > 1:
            eng.end(ids[0])
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
    per_layer = (len(ev) - 4) // n_layers
    tail = len(ev) - 2 - per_layer * n_layers             # final norm, head product (and its finish, if it is cut along K)
    if per_layer < 1 or tail < 2 or tail > 3:
        raise SystemExit(f"{len(ev)} launches were recorded: not embedding + norm + {n_layers} equal layers + 2 or 3")
    first = 2 + per_layer
    rows = ev[first:first + per_layer + 1]
    what = "decode step"
    if mixed:
        what = f"step of {B} decoded tokens beside a prompt portion of {args.portion} tokens"
    elif args.portion > 1:
        what = f"prompt step of {args.portion} tokens"
    print(f"one layer of a {what}, batch {B}, context {ctx} (times in us)")
    print(f"{'could begin':>12} {'resident before':>16} {'took':>7}  grid / block")
    base = rows[0][0]
    for (t1, t0, g, b), nxt in zip(rows[:-1], rows[1:]):
        print(f"{(t1 - base) / 1e3:12.2f} {(t1 - t0) / 1e3:16.2f} {(nxt[0] - t1) / 1e3:7.2f}  {g} / {b}")
    print(f"layer: {(rows[-1][0] - base) / 1e3:.2f} us")
    print("start and end of the step:")
    for idx in [0, 1] + list(range(len(ev) - 1 - tail, len(ev) - 1)):
        (t1, t0, g, b), nxt = ev[idx], ev[idx + 1]
        print(f"{(t1 - ev[0][0]) / 1e3:12.2f} {(t1 - t0) / 1e3:16.2f} {(nxt[0] - t1) / 1e3:7.2f}  {g} / {b}")
    print(f"step up to the sampling kernel: {(ev[-1][0] - ev[0][0]) / 1e3:.2f} us")
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--regions", type=int, default=5, help="timed regions of --steps steps each; the median is reported")
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers than the model has (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=CONTEXT)
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--skip-kernels", action="store_true", help="leave the per-kernel table out of the line")
    ap.add_argument("--decode-only", action="store_true", help="time the decode step only (for profiling a small run)")
    ap.add_argument("--prefill-only", action="store_true", help="time the 2,048-token prefill only (for profiling a small run)")
    ap.add_argument("--no-graphs", action="store_true", help="launch every kernel of a decode step one by one")
    ap.add_argument("--shape", choices=sorted(SHAPES), default=None, help="layer sizes (default llama-3-8b)")
    ap.add_argument("--workload", choices=["decode", "mixed"], default="decode",
                    help="mixed: many requests with prompts of mixed length through Runner.generate (default shape llama-3.2-1b)")
    ap.add_argument("--step-log", default=None, metavar="FILE", help="with --workload mixed: write one line per step to FILE")
    ap.add_argument("--kernels", action="store_true", help="print only the per-kernel table (decode at --batch/--context and a 2,048-token prefill)")
    ap.add_argument("--timeline", action="store_true", help="one layer of a decode step kernel by kernel (needs XRB200_TRACE=1)")
    ap.add_argument("--kernel", choices=["gemm", "attention", "sample"], default=None, help="run one kernel alone on synthetic data")
    for name, typ, default in (("tokens", int, 8), ("rows", int, 14336), ("k", int, 4096), ("splits", int, 0), ("portion", int, 1),
                               ("heads", int, 32), ("kv-heads", int, 8), ("head-dim", int, 128), ("page-size", int, 64),
                               ("vocab", int, 128256), ("iters", int, 20), ("sample-rows", int, 8)):
        ap.add_argument(f"--{name}", type=typ, default=default, help=argparse.SUPPRESS)
    ap.add_argument("--epilogue", choices=["store", "add", "swiglu"], default="store", help=argparse.SUPPRESS)
    for name in ("plain", "no-tc", "no-tma", "one-block", "spread", "mixed", "long-way", "flat"):
        ap.add_argument(f"--{name}", action="store_true", help=argparse.SUPPRESS)
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures one GPU (N=1); N={args.gpus} is not supported by this engine")
        return 2
    if args.impl == "reference":
        return reference_arm(args)
    if args.workload == "mixed":
        return mixed_workload(args)
    if args.kernel:
        return one_kernel(args)
    if args.timeline:
        return timeline(args)
    W = max(3, args.warmup)
    K = max(1, args.steps)
    R = max(1, args.regions)

    import numpy as np
    import torch
    from xyntetik_runner_b200 import kernels, measure
    from xyntetik_runner_b200.engine.engine import EngineParams, StepEntry, random_engine
    from xyntetik_runner_b200.engine.runner import EngineExecutor, Runner
    from xyntetik_runner_b200.sampling.sampler import RequestSampler, SamplingParams

    pk = measure.peaks(ROOT)
    cfg, cfgd, seed, ctx_len, shape, shape_name, full_layers = shape_config(args)
    if args.kernels:
        out = {"kernels_decode": measure.kernel_table(cfg, args.batch, ctx_len, True, pk),
               "kernels_prefill": measure.kernel_table(cfg, 2048, 2048, False, pk), "peaks": pk["source"],
               "method": "each kernel alone, CUDA events around 20 launches replayed from one CUDA graph, weights / cache layers rotated over more than L2"}
        print(json.dumps(out))
        return 0
    if args.decode_only or args.prefill_only:
        args.skip_points = args.skip_kernels = True
    kv_token_bytes = 4 * cfg.num_hidden_layers * cfg.num_key_value_heads * cfg.head_dim
    big_fits = 64 * ctx_len * kv_token_bytes <= 100e9          # batch 64 at this context within the memory left beside the weights
    max_b = args.batch if (args.skip_points or not big_fits) else max(args.batch, 64)
    t_load = time.perf_counter()
    eng = random_engine(cfg, seed, EngineParams(dtype="bfloat16", max_tokens=max_b * ctx_len, page_size=64, max_requests=max_b,
                                                max_request_tokens=ctx_len, max_step_tokens=2048,
                                                cuda_graphs=not args.no_graphs))
    for kv in eng.kv:                      # keys and values of an imagined earlier context
        kv.normal_(0.0, 1.0)
    torch.cuda.synchronize()
    load_s = time.perf_counter() - t_load
    rng = np.random.RandomState(0)
    executor = EngineExecutor(eng)
    V = cfg.vocab_size
    weight_bytes = eng.weight_bytes_per_step()
    kv_per_token = eng.kv_bytes_per_token()

    def decode_region(batch, start_len, steps, warmup):
        """Device time of `steps` decode steps of `batch` requests that already hold `start_len` tokens each (their
        keys and values are whatever the pool holds: Engine.adopt).  The event that opens the region is recorded
        behind a warm-up step that is still running, so the device is never idle inside it."""
        ids = [f"d{batch}_{i}" for i in range(batch)]
        for r in ids:
            eng.adopt(r, start_len)
        samplers = [RequestSampler(SamplingParams()) for _ in ids]
        toks = rng.randint(0, V, size=(warmup + steps, batch))
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = 0
        for s in range(warmup + steps):
            if s == warmup:
                launches0 = kernels.launch_count
                ev0.record()
            logits = eng.step([StepEntry(r, [int(toks[s, i])], [0]) for i, r in enumerate(ids)])
            executor.sampler.pick(logits, samplers)
        ev1.record()
        torch.cuda.synchronize()
        ms = ev0.elapsed_time(ev1) / steps
        launches = kernels.launch_count - launches0
        for r in ids:
            eng.end(r)
        return ms, launches

    def decode_point(batch, start_len, steps, warmup, regions):
        runs = [decode_region(batch, start_len, steps, warmup) for _ in range(regions)]
        ms = statistics.median(m for m, _ in runs)
        nbytes = weight_bytes + batch * (start_len + warmup + steps / 2.0) * kv_per_token
        gbs = nbytes / (ms * 1e-3) / 1e9
        return {"tok_s": batch * 1e3 / ms, "ms": ms, "ms_min": min(m for m, _ in runs), "ms_max": max(m for m, _ in runs),
                "bytes": int(nbytes), "gbs": gbs, "frac": gbs / pk["hbm_gbs"], "launches": runs[0][1]}

    def through_entry_point(batch, prompt_len, steps, warmup):
        """`batch` real prompts of `prompt_len` random tokens through Runner.generate (the public API and nothing else):
        the scheduler cuts the prompts into portions, admits, decodes; every step the host sends the step's token ids
        and block-table rows (pinned memory, one copy) and reads the sampled ids back.  Requests finish their prompts
        at different steps, so the timed window is `steps` steps of the LAST request to start decoding, while every
        request is decoding: from the arrival of its token `warmup` to that of its token `warmup + steps`."""
        runner = Runner(engine=eng)
        budget = runner.scheduler.params.max_step_tokens
        spread = -(-batch * prompt_len // budget) + batch + 2          # steps between the first and the last request's first token
        n_new = warmup + steps + spread + 2
        prompts = [[int(t) for t in rng.randint(0, V, size=prompt_len)] for _ in range(batch)]
        stamps = {}
        marks = {}

        def on_token(rid, tok, done):
            lst = stamps.setdefault(rid, [])
            lst.append(time.perf_counter())
            if len(lst) in (warmup + 1, warmup + steps + 1):
                marks[rid, len(lst)] = (eng.h2d_bytes, runner.scheduler.stats["steps"])
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        res = runner.generate(prompts, n=n_new, ignore_eos=True, on_token=on_token)
        last = max(stamps, key=lambda r: stamps[r][0])                   # the request whose first token came last
        ts = stamps[last]
        wall = ts[warmup + steps] - ts[warmup]
        h2d = (marks[last, warmup + steps + 1][0] - marks[last, warmup + 1][0]) / steps
        n_steps = marks[last, warmup + steps + 1][1] - marks[last, warmup + 1][1]
        all_decoding = all(len(stamps[r]) >= 1 and stamps[r][0] <= ts[warmup] and len(r_.tokens) == n_new
                           for r, r_ in zip(sorted(stamps), res)) and n_steps == steps
        first_token_s = min(s[0] for s in stamps.values()) - t0
        return {"ms": wall * 1e3 / steps, "tok_s": batch * steps / wall, "h2d": h2d, "valid": bool(all_decoding),
                "prompt_tok_s_first": prompt_len / first_token_s if batch == 1 else None, "context_mid": prompt_len + warmup + spread // 2 + steps // 2}

    def prefill(T, reps):
        ms = []
        for rep in range(reps + 2):
            toks = [int(t) for t in rng.randint(0, V, size=T)]
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            ev0.record()
            eng.step([StepEntry("p", toks, [T - 1])])
            ev1.record()
            torch.cuda.synchronize()
            eng.end("p")
            if rep >= 2:
                ms.append(ev0.elapsed_time(ev1))
        L, d, H, Kh, hd, F = cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.intermediate_size
        flops = 2.0 * T * L * (d * (H + 2 * Kh) * hd + H * hd * d + 3 * d * F) + 2.0 * d * V + L * 4.0 * H * hd * (T * (T + 1) / 2)
        m = statistics.median(ms)
        return {"value": T * 1e3 / m, "tokens": T, "ms": m, "ms_min": min(ms), "ms_max": max(ms),
                "frac": flops / (m * 1e-3) / (pk["bf16_tflops"] * 1e12),
                "frac_of_sustained": flops / (m * 1e-3) / (pk.get("bf16_tflops_sustained", pk["bf16_tflops"]) * 1e12)}

    clocks = ClockSampler()
    clocks.start()
    start_len = ctx_len - (W + K) - 2
    if args.prefill_only:
        pre = prefill(2048, max(3, W))
        clocks.stop()
        print(json.dumps({"prefill_only": True, "tokens": 2048, "ms": pre["ms"], "tok_s": pre["value"]}))
        return 0
    decode_region(args.batch, start_len, min(8, K), min(8, W))          # untimed: clocks and caches as in the middle of a run
    head = decode_point(args.batch, start_len, K, W, R)
    if args.decode_only:
        clocks.stop()
        print(json.dumps({"decode_only": True, "batch": args.batch, "context": ctx_len, "ms_per_step": head["ms"],
                          "tok_s": head["tok_s"], "launches": head["launches"]}))
        return 0
    spread = -(-args.batch * ctx_len // 2048) + args.batch + 2
    e2e = through_entry_point(args.batch, ctx_len - (W + K + spread + 2) - 2, K, W)
    pre = prefill(2048, max(3, W))
    points, e2e_points = {}, {}
    if not args.skip_points:
        short = max(16, K // 2)
        for b in (1, 64) if big_fits else (1,):
            points[f"decode_b{b}"] = decode_point(b, ctx_len - (W + short) - 2, short, W, 3)
        for b in (1, 8, 64):          # the reference workload: 512-token prompts, 256 generated (mid-point 640)
            if b <= max_b:
                points[f"decode_b{b}_ctx640"] = decode_point(b, 640 - W - short // 2, short, W, 3)
        points["prefill_512"] = prefill(512, 3)
        for b in (1, 8, 64):          # ... and through the entry point: real 512-token prompts, decode rate while all decode
            if b <= max_b:
                r = through_entry_point(b, 512, min(K, 128), W)
                e2e_points[f"b{b}"] = {"decode_tok_s": r["tok_s"], "ms_per_step": r["ms"], "valid": r["valid"],
                                       "prompt_tok_s": r["prompt_tok_s_first"]}
    kern = {}
    if not args.skip_kernels:
        kern = {"decode": measure.kernel_table(cfg, args.batch, ctx_len, True, pk),
                "prefill_2048": measure.kernel_table(cfg, 2048, 2048, False, pk)}
    clk = clocks.stop()

    L, d, H, Kh, hd, F = cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.intermediate_size
    line = {
        "metric": f"decode tok/s at batch {args.batch} ({shape_name} shape, bf16, context {ctx_len})",
        "value": head["tok_s"], "unit": "tok/s",
        "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": head["ms"], "ms_per_step_min": head["ms_min"], "ms_per_step_max": head["ms_max"],
        "regions": R, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": f"synthetic (random weights seed {seed}, random token ids, random cached keys/values)",
        "config": {"model": shape + "-shape", "layers": cfg.num_hidden_layers, "layers_of_model": full_layers,
                   "hidden": d, "heads": H, "kv_heads": Kh, "head_dim": hd, "intermediate": F, "vocab": V,
                   "global_batch": args.batch, "seq_len": ctx_len, "page_size": 64, "parallelism": "single-gpu",
                   "l2": "step inputs (weights) exceed L2", "peaks": pk["source"], "timing": f"median of {R} regions of {K} steps"},
        "e2e": {"value": e2e["tok_s"], "unit": "tok/s", "h2d_bytes_per_step": int(e2e["h2d"]), "d2h_bytes_per_step": 4 * args.batch,
                "ms_per_step": e2e["ms"], "valid": e2e["valid"], "context_mid": e2e["context_mid"],
                "path": "Runner.generate(real prompts of context length) -> Scheduler.step (next decode step launched ahead) -> Engine.step "
                        "-> DeviceSampler -> host ids",
                "note": f"wall clock between the arrivals of tokens {W} and {W + K} of the last request to start decoding, all {args.batch} decoding"},
        "gpu_launches": head["launches"],
        "prefill": pre,
        "roofline": {"bound": "hbm", "achieved": head["gbs"], "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": head["frac"]},
        "points": {k: (v["tok_s"] if "tok_s" in v else v["value"]) for k, v in points.items()},
        "points_detail": {k: {kk: v[kk] for kk in ("ms", "bytes", "gbs", "frac") if kk in v} for k, v in points.items()},
        "e2e_points": e2e_points,
        "kernels": kern,
        "clocks": clk,
        "load_s": load_s,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
