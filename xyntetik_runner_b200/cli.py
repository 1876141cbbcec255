"""The command line, in the reference's manner (`runner -m MODEL -p TEXT -n N --temp F`, src/main.c:188-340).

Options keep the reference's names and meanings where it has them: -m (here a model FOLDER with
config.json and model.safetensors), -p, -f, -n (default 256, -1 = until a stop id), -c, -b, -s (0 is
refused), --temp (0 = greedy), --top-k, --top-p, --min-p, --repeat-penalty, --ignore-eos, --no-bos,
--score (teacher-forced log-probabilities of the prompt, the reference's JSON), --parallel, --rope-base, --rope-scale,
--bench-json (extended: --parallel sequences at once and a per-kernel table), -t, -v/--version; -c 0 fits the context
to the free memory.  Where the reference has --gpu off to run its CPU code, --ref runs the plain implementation
that the tests compare the engine with (greedy only; it is slow and is found only in a source checkout).  Tokenisation is outside the engine: a prompt is either ``ids:1,2,3`` (or a file of
ids, --prompt-ids) or
text taken byte by byte (token id = byte value), and the output is printed as ids (and as bytes where
every id is one).
"""
from __future__ import annotations

import argparse
import json
import sys
import time

from . import __version__


def unescape(s: str) -> str:
    """\\n \\t \\r \\\\ in a -p argument (src/main.c:168-186)."""
    out, i = [], 0
    while i < len(s):
        if s[i] == "\\" and i + 1 < len(s) and s[i + 1] in "ntr\\":
            out.append({"n": "\n", "t": "\t", "r": "\r", "\\": "\\"}[s[i + 1]])
            i += 2
        else:
            out.append(s[i])
            i += 1
    return "".join(out)


def encode_prompt(text: str, vocab: int):
    if text.startswith("ids:"):
        try:
            ids = [int(t) for t in text[4:].replace(" ", "").split(",") if t != ""]
        except ValueError:
            raise SystemExit("error: -p ids:... must be a comma-separated list of integers")
    else:
        ids = list(text.encode("utf-8"))
    bad = [t for t in ids if t < 0 or t >= vocab]
    if bad:
        raise SystemExit(f"error: token id {bad[0]} is outside the vocabulary of {vocab}")
    return ids


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="runner", description="generate with a dense Llama model on one B200")
    ap.add_argument("-m", dest="model", help="model folder (config.json + model.safetensors)")
    ap.add_argument("-p", dest="prompt", default=None, help="prompt: text (bytes) or ids:1,2,3; \\n etc. are unescaped")
    ap.add_argument("-f", dest="file", default=None, help="read prompt from file (appended after -p text)")
    ap.add_argument("--prompt-ids", default=None, metavar="FILE",
                    help="read the prompt as token ids from FILE (integers separated by commas or white space); instead of -p / -f")
    ap.add_argument("-n", dest="n", type=int, default=256, help="max tokens to generate (default 256, -1 = until a stop id)")
    ap.add_argument("-c", dest="ctx", type=int, default=None,
                    help="context length (default: min(model max, 4096); 0 = as long as the model allows and memory holds)")
    ap.add_argument("-t", dest="threads", type=int, default=None, help="CPU threads (used by --ref only: the engine computes on the GPU)")
    ap.add_argument("--ref", action="store_true",
                    help="generate greedily with the plain CPU implementation under tests/ instead of the engine (for comparison)")
    ap.add_argument("-b", dest="batch", type=int, default=2048, help="prompt portion / step token budget (default 2048)")
    ap.add_argument("-s", dest="seed", type=int, default=None, help="RNG seed (default: time; 0 is refused)")
    ap.add_argument("--temp", type=float, default=0.0, help="temperature (0 = greedy: the argmax, no repeat penalty)")
    ap.add_argument("--top-k", type=int, default=0, help="top-k (0 = off)")
    ap.add_argument("--top-p", type=float, default=1.0, help="top-p")
    ap.add_argument("--min-p", type=float, default=0.0, help="min-p vs the top candidate (0 = off)")
    ap.add_argument("--repeat-penalty", type=float, default=1.0, help="penalty on recently emitted tokens (1 = off)")
    ap.add_argument("--ignore-eos", action="store_true", help="keep generating past stop ids")
    ap.add_argument("--score", action="store_true",
                    help="teacher-forced scoring: per-token log P(token|prefix) of the prompt as JSON; nothing is generated")
    ap.add_argument("--parallel", type=int, default=1, help="request slots of the engine (default 1)")
    ap.add_argument("--rope-base", type=float, default=None, help="override rope frequency base")
    ap.add_argument("--rope-scale", type=float, default=None, help="force linear rope position scaling by F")
    ap.add_argument("--no-bos", action="store_true", help="do not prepend the BOS token")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16",
                    help="bfloat16: serving kernels; float32: everything in true 32 bit")
    ap.add_argument("--page-size", type=int, default=64, help="tokens per cache page")
    ap.add_argument("--bench-json", action="store_true",
                    help="prefill 512-token prompts (--parallel of them at once), decode -n tokens each with stop ids ignored, "
                         "print timings and a per-kernel table as JSON")
    ap.add_argument("--random", type=int, default=None, metavar="SEED",
                    help="with -m: write config.json-described random weights into the folder first (needs config.json)")
    ap.add_argument("-v", "--version", action="version", version=f"runner-b200 {__version__}")
    return ap


def run_plain(args) -> int:
    """--ref: the plain implementation of the tests (whole sequences on the CPU, no cache), greedy decoding."""
    import os
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    tests = os.path.join(here, "tests")
    if not os.path.isfile(os.path.join(tests, "plain_llama.py")):
        print("error: --ref needs tests/plain_llama.py of a source checkout", file=sys.stderr)
        return 2
    if args.temp > 0 or args.score or args.bench_json:
        print("error: --ref decodes greedily only (no --temp, --score or --bench-json)", file=sys.stderr)
        return 2
    if args.threads:
        import torch
        torch.set_num_threads(args.threads)
        os.environ["OMP_NUM_THREADS"] = str(args.threads)
    sys.path.insert(0, tests)
    from plain_llama import PlainLlama
    m = PlainLlama(args.model)
    text = unescape(args.prompt) if args.prompt is not None else ""
    if args.file:
        with open(args.file, "r", encoding="utf-8") as f:
            text += f.read()
    ids = encode_prompt(text, m.cfg["vocab_size"])
    bos = m.cfg.get("bos_token_id")
    if not args.no_bos and bos is not None:
        ids = [int(bos)] + ids
    if not ids:
        print("error: empty prompt", file=sys.stderr)
        return 2
    stops = m.cfg.get("eos_token_id")
    stops = set() if (stops is None or args.ignore_eos) else set(stops if isinstance(stops, list) else [stops])
    out = []
    for _ in range(args.n if args.n > 0 else 256):
        tok = m.generate_greedy(ids + out, 1)[0]
        if tok in stops:
            break
        out.append(tok)
    print("ids:" + ",".join(str(t) for t in out))
    return 0


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if not args.model:
        print("error: -m MODEL is required", file=sys.stderr)
        return 2
    if args.seed is not None and args.seed == 0:
        print("error: -s 0 is refused (it is the generator's fixed point); pick another seed", file=sys.stderr)
        return 2
    if args.random is not None:
        import os
        import torch
        from .config import registry
        from .weights.loader import write_model_folder
        from . import architectures  # noqa: F401
        arch, cfg = registry.load_config(args.model)
        specs = arch.build_plan(cfg).tensor_specs()
        dt = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float32}[cfg.torch_dtype]
        write_model_folder(args.model, cfg.to_dict(), specs, args.random, dt)
        print(f"wrote random weights (seed {args.random}) to {os.path.join(args.model, 'model.safetensors')}", file=sys.stderr)
        if args.prompt is None and args.file is None and not args.bench_json:
            return 0
    if args.ref:
        return run_plain(args)
    from .engine.runner import Runner
    t0 = time.perf_counter()
    if args.parallel < 1 or (args.rope_base is not None and not args.rope_base > 0) or \
            (args.rope_scale is not None and not args.rope_scale > 0):
        print("error: --parallel needs N >= 1, --rope-base a positive base, --rope-scale a positive factor", file=sys.stderr)
        return 2
    runner = Runner(args.model, dtype=args.dtype, ctx=args.ctx, batch=args.batch, parallel=args.parallel,
                    page_size=args.page_size, rope_base=args.rope_base, rope_scale=args.rope_scale)
    plan = runner.engine.plan
    print(f"loaded {args.model} in {time.perf_counter() - t0:.2f} s ({args.dtype})", file=sys.stderr)
    if args.bench_json:
        # the reference's --bench-json (src/main.c:1435-1515): prompt_tok_s, gen_tok_s, prompt_s, gen_s of a 512-token
        # prompt and -n decoded tokens; here for --parallel sequences at once, with the kernels' own times beside them
        import numpy as np
        from . import measure
        B = args.parallel
        rng = np.random.RandomState(0)
        prompts = [[int(t) for t in rng.randint(0, plan.vocab_size, size=512)] for _ in range(B)]
        n_new = args.n if args.n > 0 else 128
        first, last = {}, {}

        def on_token(rid, tok, done):
            first.setdefault(rid, time.perf_counter())
            last[rid] = time.perf_counter()
        t0 = time.perf_counter()
        res = runner.generate(prompts, n=n_new, temp=args.temp, seed=args.seed, ignore_eos=True, on_token=on_token)
        t_first, t_last = max(first.values()), max(last.values())          # every prompt is in; every sequence is done
        prompt_s, gen_s = t_first - t0, t_last - t_first
        gen = sum(len(r.tokens) for r in res)
        out = {"batch": B, "prompt_tokens": 512 * B, "gen_tokens": gen, "prompt_s": prompt_s, "gen_s": gen_s,
               "prompt_tok_s": 512 * B / prompt_s, "gen_tok_s": (gen - B) / gen_s if gen_s > 0 else 0.0,
               "dtype": args.dtype, "steps": runner.scheduler.stats.get("steps")}
        cfg = runner.engine.config
        if args.dtype == "bfloat16" and all(hasattr(cfg, k) for k in ("hidden_size", "num_attention_heads", "num_key_value_heads",
                                                                      "head_dim", "intermediate_size", "vocab_size")):
            del runner
            out["kernels"] = measure.kernel_table(cfg, B, 512 + n_new // 2, True, measure.peaks(), iters=10)
        print(json.dumps(out))
        return 0
    if args.prompt_ids is not None:
        if args.prompt is not None or args.file:
            print("error: --prompt-ids stands instead of -p and -f", file=sys.stderr)
            return 2
        with open(args.prompt_ids, "r", encoding="utf-8") as f:
            ids = encode_prompt("ids:" + ",".join(f.read().replace(",", " ").split()), plan.vocab_size)
    else:
        text = unescape(args.prompt) if args.prompt is not None else ""
        if args.file:
            with open(args.file, "r", encoding="utf-8") as f:
                text += f.read()
        ids = encode_prompt(text, plan.vocab_size)
    if not args.no_bos and plan.bos_id is not None:
        ids = [plan.bos_id] + ids
    if not ids:
        print("error: empty prompt", file=sys.stderr)
        return 2
    if args.score:
        # the reference's --score output (src/main.c:1377-1428)
        import math
        try:
            lps = runner.score(ids, portion=min(args.batch, 256))
        except ValueError as e:
            print(f"error: --score: {e}", file=sys.stderr)
            return 2
        nll = -sum(lps)
        mean = nll / len(lps)
        print(json.dumps({"schema_version": "xyntetik.runner.score.v1", "n_tokens": len(ids), "n_scored": len(lps), "tokens": ids,
                          "logprobs": [float(f"{x:.9g}") for x in lps], "nll_total": float(f"{nll:.9g}"),
                          "nll_mean": float(f"{mean:.9g}"), "ppl": float(f"{math.exp(mean):.9g}")}))
        return 0
    t0 = time.perf_counter()
    first = {}
    def on_token(rid, tok, done):
        first.setdefault("t", time.perf_counter())
    try:
        res = runner.generate(ids, n=args.n, temp=args.temp, top_k=args.top_k, top_p=args.top_p, min_p=args.min_p,
                              repeat_penalty=args.repeat_penalty, seed=args.seed, ignore_eos=args.ignore_eos,
                              on_token=on_token)
    except ValueError as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    t1 = time.perf_counter()
    print("ids:" + ",".join(str(t) for t in res.tokens))
    if res.tokens and all(0 <= t < 256 for t in res.tokens):
        sys.stdout.buffer.write(bytes(res.tokens) + b"\n")
    tp = first.get("t", t1) - t0
    tg = t1 - first.get("t", t1)
    print(f"prompt: {len(ids)} tokens, {len(ids) / tp if tp > 0 else 0:.1f} tok/s | gen: {len(res.tokens)} tokens, "
          f"{(len(res.tokens) - 1) / tg if tg > 0 else 0:.1f} tok/s | finish: {res.finish_reason}", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
