#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Llama-3-8B shape, random weights, one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl reference]
    python bench.py --shape llama-2-13b --context 3840      # the same measurement at another shape of the architecture
    python bench.py --workload mixed                        # 64 requests of 16..4,096 tokens through Runner.generate

A "step" is one decode step of the whole batch through the engine's step function and the device
sampler.  One JSON line is printed: `value` = decoded tokens per second at batch 8 with every request
at the benchmark context (device-timed with CUDA events over exactly K steps); `e2e` = the same rate
through the Python entry point's loop (host token ids in, sampled ids back to the host every step);
`prefill` = a 2,048-token prompt in one step; `roofline` = bytes the decode step must read (every
weight once + the live requests' keys and values) / its time / the measured copy bandwidth; `points` =
decode at batch 1 and 64.  This program measures one GPU only.
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
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        try:
            with open(p) as f:
                d = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if isinstance(d.get(k), (int, float)) and d[k] > 0:
                    out[k] = float(d[k])
            out["source"] = "measured"
            return out
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


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
               "step_token_budget": 2048}
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


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers than the model has (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=CONTEXT)
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--decode-only", action="store_true", help="time the decode step only (for profiling a small run)")
    ap.add_argument("--prefill-only", action="store_true", help="time the 2,048-token prefill only (for profiling a small run)")
    ap.add_argument("--no-graphs", action="store_true", help="launch every kernel of a decode step one by one")
    ap.add_argument("--shape", choices=sorted(SHAPES), default=None, help="layer sizes (default llama-3-8b)")
    ap.add_argument("--workload", choices=["decode", "mixed"], default="decode",
                    help="mixed: many requests with prompts of mixed length through Runner.generate (default shape llama-3.2-1b)")
    ap.add_argument("--step-log", default=None, metavar="FILE", help="with --workload mixed: write one line per step to FILE")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a C program without a Python package at its root; pip install of it fails offline, "
                          "and it reads GGUF files only (no bf16 Llama-3-8B GGUF can be had without network)"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU (N=1); N={args.gpus} is not supported by this engine")
        return 2
    if args.workload == "mixed":
        return mixed_workload(args)
    W = max(3, args.warmup)
    K = max(1, args.steps)

    import numpy as np
    import torch
    from xyntetik_runner_b200 import kernels
    from xyntetik_runner_b200.config.llama import LlamaConfig
    from xyntetik_runner_b200.engine.engine import EngineParams, StepEntry, random_engine
    from xyntetik_runner_b200.engine.runner import EngineExecutor
    from xyntetik_runner_b200.engine.scheduler import Request, Scheduler, SchedulerParams
    from xyntetik_runner_b200.sampling.sampler import RequestSampler, SamplingParams

    pk = peaks()
    shape = args.shape or "llama-3-8b"
    shape_cfg, seed, shape_ctx, shape_name = SHAPES[shape]
    full_layers = shape_cfg["num_hidden_layers"]
    if args.shape is not None and args.layers == FULL_LAYERS:
        args.layers = full_layers
    if args.shape is not None and args.context == CONTEXT:
        args.context = shape_ctx
    cfgd = dict(shape_cfg, num_hidden_layers=args.layers, max_position_embeddings=max(shape_cfg["max_position_embeddings"], args.context))
    cfg = LlamaConfig.from_dict(cfgd)
    if args.decode_only or args.prefill_only:
        args.skip_points = True
    ctx_len = args.context
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

    def decode_run(batch, start_len, steps, warmup, e2e=False):
        """Times `steps` decode steps of `batch` requests that already hold `start_len` tokens each."""
        ids = [f"d{batch}_{i}" for i in range(batch)]
        for r in ids:
            eng.adopt(r, start_len)
        samplers = [RequestSampler(SamplingParams()) for _ in ids]
        toks = rng.randint(0, V, size=(warmup + steps, batch))
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        last = [int(t) for t in toks[0]]
        launches0 = h2d = d2h = 0
        t_wall = 0.0
        for s in range(warmup + steps):
            if s == warmup:
                torch.cuda.synchronize()
                launches0 = kernels.launch_count
                t_wall = time.perf_counter()
                ev0.record()
            if e2e:
                entries = [StepEntry(r, [last[i]], [0]) for i, r in enumerate(ids)]
                logits = eng.step(entries)
                last = executor.sampler.pick(logits, samplers).cpu().tolist()      # sampled ids back on the host
            else:
                entries = [StepEntry(r, [int(toks[s, i])], [0]) for i, r in enumerate(ids)]
                logits = eng.step(entries)
                executor.sampler.pick(logits, samplers)
        ev1.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t_wall
        ms = ev0.elapsed_time(ev1) / steps
        launches = kernels.launch_count - launches0
        for r in ids:
            eng.end(r)
        return {"ms": ms, "wall_ms": wall * 1e3 / steps, "launches": launches}

    def e2e_run_through_entry_point(batch, start_len, steps, warmup):
        """The same decode steps through the Python entry point's own loop (Runner -> Scheduler -> Engine.step ->
        device sampler): every step the host sends that step's token ids and block-table rows (pinned memory,
        one copy) and reads the sampled ids back.  The requests enter with `start_len` tokens of context already
        in the cache (Engine.adopt), so that the timed region is decoding at the benchmark context."""
        from xyntetik_runner_b200.engine.runner import Runner
        runner = Runner(engine=eng)
        sch = runner.scheduler
        sch.params.max_step_tokens = max(sch.params.max_step_tokens, batch)
        for i in range(batch):
            rid = f"e{i}"
            req = Request(rid, [int(t) for t in rng.randint(0, V, size=start_len + 1)], max_new_tokens=warmup + steps,
                          sampling=SamplingParams(), ignore_eos=True)
            sch.add(req)
            sch.waiting.remove(req)
            eng.adopt(rid, start_len)            # context in the cache without paying for its prefill
            req.computed, req.status, req.admitted_at = start_len, "live", i
            sch.live.append(req)
        h2d0 = eng.h2d_bytes
        for s in range(warmup):
            sch.step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        h2d1 = eng.h2d_bytes
        n_tok = 0
        for s in range(steps):
            n_tok += sum(1 for _, tok, _ in sch.step() if tok is not None)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        h2d = (eng.h2d_bytes - h2d1) / steps
        while sch.has_work():
            sch.step()
        for i in range(batch):
            sch.finished.pop(f"e{i}", None)
        return {"wall_ms": wall * 1e3 / steps, "tokens": n_tok, "h2d": h2d}

    clocks = ClockSampler()
    clocks.start()
    start_len = ctx_len - (W + K) - 2
    if not args.prefill_only:
        decode_run(args.batch, start_len, 8, 8)          # untimed: clocks and caches as in the middle of a run
    main_run = decode_run(args.batch, start_len, K, W) if not args.prefill_only else None
    if args.decode_only:
        clocks.stop()
        print(json.dumps({"decode_only": True, "batch": args.batch, "context": ctx_len, "ms_per_step": main_run["ms"],
                          "tok_s": args.batch * 1e3 / main_run["ms"], "launches": main_run["launches"]}))
        return 0
    e2e_run = e2e_run_through_entry_point(args.batch, start_len, K, W) if not args.prefill_only else None
    assert args.prefill_only or e2e_run["tokens"] == args.batch * K

    # prefill of 2,048 tokens in one step
    T = 2048
    pre_ms = []
    for rep in range(W + 3):
        toks = [int(t) for t in rng.randint(0, V, size=T)]
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        ev0.record()
        eng.step([StepEntry("p", toks, [T - 1])])
        ev1.record()
        torch.cuda.synchronize()
        eng.end("p")
        if rep >= W:
            pre_ms.append(ev0.elapsed_time(ev1))
    pre = statistics.median(pre_ms)
    if args.prefill_only:
        clocks.stop()
        print(json.dumps({"prefill_only": True, "tokens": T, "ms": pre, "tok_s": T * 1e3 / pre}))
        return 0
    L, d, H, Kh, hd, F = cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.intermediate_size
    gemm_flops = 2.0 * T * L * (d * (H + 2 * Kh) * hd + H * hd * d + 3 * d * F) + 2.0 * d * V
    attn_flops = L * 4.0 * H * hd * (T * (T + 1) / 2)
    pre_flops = gemm_flops + attn_flops

    points = {}
    if not args.skip_points:
        for b in (1, 64) if big_fits else (1,):
            r = decode_run(b, start_len, max(4, K // 2), W)
            points[f"decode_b{b}"] = b * 1e3 / r["ms"]
        for b in (1, 8, 64):          # the reference workload: 512-token prompts, 256 generated (mid-point 640)
            if b > max_b:
                continue
            r = decode_run(b, 640 - W - max(4, K // 2), max(4, K // 2), W)
            points[f"decode_b{b}_ctx640"] = b * 1e3 / r["ms"]
    clk = clocks.stop()

    ms = main_run["ms"]
    value = args.batch * 1e3 / ms
    kv_bytes = args.batch * (start_len + W + K / 2.0) * eng.kv_bytes_per_token()
    step_bytes = eng.weight_bytes_per_step() + kv_bytes
    achieved = step_bytes / (ms * 1e-3) / 1e9
    line = {
        "metric": f"decode tok/s at batch {args.batch} ({shape_name} shape, bf16, context {ctx_len})",
        "value": value, "unit": "tok/s",
        "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": f"synthetic (random weights seed {seed}, random token ids, random cached keys/values)",
        "config": {"model": shape + "-shape", "layers": cfg.num_hidden_layers, "layers_of_model": full_layers,
                   "hidden": d, "heads": H, "kv_heads": Kh, "head_dim": hd, "intermediate": F, "vocab": V,
                   "global_batch": args.batch, "seq_len": ctx_len, "page_size": 64, "parallelism": "single-gpu",
                   "l2": "step inputs (weights) exceed L2", "peaks": pk["source"]},
        "e2e": {"value": args.batch * 1e3 / e2e_run["wall_ms"], "unit": "tok/s",
                "h2d_bytes_per_step": int(e2e_run["h2d"] + 24 * args.batch),      # step description + sampling parameters
                "d2h_bytes_per_step": 4 * args.batch, "ms_per_step": e2e_run["wall_ms"],
                "path": "Runner -> Scheduler.step (next decode step launched ahead) -> Engine.step -> DeviceSampler -> host ids",
                "note": "the timed region holds exactly K steps of device work: one step is in flight when it starts and one when it ends"},
        "gpu_launches": main_run["launches"],
        "prefill": {"value": T * 1e3 / pre, "tokens": T, "ms": pre, "frac": pre_flops / (pre * 1e-3) / (pk["bf16_tflops"] * 1e12),
                    "frac_of_sustained": pre_flops / (pre * 1e-3) / (pk.get("bf16_tflops_sustained", pk["bf16_tflops"]) * 1e12)},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"]},
        "points": points,
        "clocks": clk,
        "load_s": load_s,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
