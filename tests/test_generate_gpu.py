"""Generation through the Python entry point and the command line, against the plain implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import tiny
import traces
from plain_llama import PlainLlama, sample_chain, uniform_from_state, xorshift64

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {(n, dt): tiny.make_folder(str(tmp_path_factory.mktemp(f"g{n}{dt}")), n, dt)
            for n in "AB" for dt in ("float32", "bfloat16")}


def check_against_plain(plain, prompt, generated, temp, seed, tol, **chain):
    """Teacher-forced: every generated token must be what the plain implementation picks for the same
    prefix and the same draw.  Where it is not, the draw must lie within `tol` of the token's interval of
    the plain cumulative distribution (greedy: the token's plain logit within `tol` of the best): the
    engine's logits differ from the plain ones by rounding, which moves the intervals' edges a little.
    Returns the number of tokens that differed."""
    state = seed
    differed = 0
    for i, tok in enumerate(generated):
        lg = plain.logits(list(prompt) + list(generated[:i]))[-1]
        r = 0.0
        if temp > 0:
            state = xorshift64(state)
            r = uniform_from_state(state)
        pick = sample_chain(lg, r, temp, **chain)
        if pick != tok:
            dist = sample_chain(lg, r, temp, distance_of=tok, **chain)
            assert dist <= tol, f"token {i}: engine {tok}, plain {pick}; the draw is {dist:.3e} outside the token's interval"
            differed += 1
    return differed


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_workload_a_greedy(folders, dtype):
    """Three requests, prompts of 5/11/17 tokens, 16 greedy steps each, pages of 16."""
    from xyntetik_runner_b200.engine.runner import Runner
    folder = folders["A", dtype]
    plain = PlainLlama(folder)
    prompts = [traces.random_tokens(i, n, 256) for i, n in enumerate((5, 11, 17))]
    r = Runner(folder, dtype=dtype, ctx=128, parallel=3, page_size=16)
    res = r.generate(prompts, n=16, temp=0.0, ignore_eos=True)
    for p, g in zip(prompts, res):
        assert len(g.tokens) == 16 and g.finish_reason == "length"
        if dtype == "float32":
            assert g.tokens == plain.generate_greedy(p, 16)
        else:
            assert check_against_plain(plain, p, g.tokens, 0.0, 0, tol=0.05) <= 2
    r.engine.cache.audit()
    assert not r.engine.cache.live_requests()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_workload_b_temperature_chunked(folders, dtype):
    """Four requests, prompts of 1/9/33/70 tokens, prefill in portions of 24 mixed with decoding, 20 steps at
    temperature 0.8 with fixed seeds, pages of 8."""
    from xyntetik_runner_b200.engine.runner import Runner
    folder = folders["B", dtype]
    plain = PlainLlama(folder)
    prompts = [traces.random_tokens(10 + i, n, 387) for i, n in enumerate((1, 9, 33, 70))]
    r = Runner(folder, dtype=dtype, ctx=128, parallel=4, page_size=8, batch=40, prefill_chunk=24)
    res = r.generate(prompts, n=20, temp=0.8, seed=77, ignore_eos=True)
    assert r.scheduler.stats["max_batch"] >= 3
    # float32 logits agree to ~1e-5, which moves an edge of the cumulative distribution by less than 1e-4;
    # bfloat16 logits carry ~1% error, and the edges move by about as much
    tol = 1e-4 if dtype == "float32" else 2e-2
    for i, (p, g) in enumerate(zip(prompts, res)):
        assert len(g.tokens) == 20
        differed = check_against_plain(plain, p, g.tokens, 0.8, 77 + i, tol=tol)
        assert dtype != "float32" or differed == 0
    # the same seeds give the same tokens whatever the batching
    r2 = Runner(folder, dtype=dtype, ctx=128, parallel=1, page_size=64)
    for i, (p, g) in enumerate(zip(prompts, res)):
        alone = r2.generate(p, n=20, temp=0.8, seed=77 + i, ignore_eos=True)
        if dtype == "float32":
            assert alone.tokens == g.tokens


def test_full_chain_options(folders):
    from xyntetik_runner_b200.engine.runner import Runner
    folder = folders["B", "float32"]
    plain = PlainLlama(folder)
    p = traces.random_tokens(3, 12, 387)
    r = Runner(folder, dtype="float32", ctx=128, parallel=1, page_size=8)
    g = r.generate(p, n=24, temp=1.3, top_k=40, top_p=0.9, min_p=0.02, repeat_penalty=1.3, seed=9, ignore_eos=True)
    # the plain chain needs the penalty window: prompt and generated tokens so far
    state = 9
    for i, tok in enumerate(g.tokens):
        lg = plain.logits(p + g.tokens[:i])[-1]
        state = xorshift64(state)
        pick, margin = sample_chain(lg, uniform_from_state(state), 1.3, top_k=40, top_p=0.9, min_p=0.02,
                                    repeat_penalty=1.3, recent=(p + g.tokens[:i])[-256:], with_margin=True)
        assert pick == tok or margin < 1e-4, (i, tok, pick, margin)


def test_stop_ids_end_a_request(folders):
    from xyntetik_runner_b200.engine.runner import Runner
    folder = folders["A", "float32"]
    plain = PlainLlama(folder)
    p = traces.random_tokens(8, 9, 256)
    free = plain.generate_greedy(p, 12)
    r = Runner(folder, dtype="float32", ctx=128, parallel=1, page_size=16)
    rid = r.submit(p, n=12, stop_ids=[free[5]])
    while r.scheduler.has_work():
        r.scheduler.step()
    q = r.scheduler.finished[rid]
    first = free.index(free[5])
    assert q.finish_reason == "stop" and q.generated == free[:first]


def test_callback_ends_a_request(folders):
    """on_token returning False ends that request at once (reason "abort"); the request beside it goes on unchanged,
    also while steps are launched ahead."""
    from xyntetik_runner_b200.engine.runner import Runner
    folder = folders["A", "float32"]
    plain = PlainLlama(folder)
    pa, pb = traces.random_tokens(21, 9, 256), traces.random_tokens(22, 14, 256)
    want_a, want_b = plain.generate_greedy(pa, 10), plain.generate_greedy(pb, 10)
    r = Runner(folder, dtype="float32", ctx=128, parallel=2, page_size=16)
    seen = {0: 0, 1: 0}

    def on_token(rid, tok, done):
        seen[rid] += 1
        return not (rid == 0 and seen[0] == 4)           # the first request is ended when its 4th token arrives

    a, b = r.generate([pa, pb], n=10, temp=0.0, ignore_eos=True, on_token=on_token)
    assert a.finish_reason == "abort" and a.tokens == want_a[:4]
    assert b.finish_reason == "length" and b.tokens == want_b
    assert not r.engine.cache.live_requests()
    r.engine.cache.audit()


@pytest.mark.parametrize("temp,penalty", [(0.0, 1.0), (0.9, 1.0), (1.4, 1.5)])
def test_steps_launched_ahead_give_the_same_tokens(folders, temp, penalty):
    """Decode steps launched before the tokens of the step ahead of them are read (the device feeds the sampled ids
    on) against the same run one step at a time: requests of different lengths, one that meets a stop token.  With
    a repeat penalty the window of recent tokens lacks, on the host, the token that is still on the device: the kernel
    puts it in (unless it is one of the request's stop ids, which a window never holds: the last request goes on
    after its stop ids with `ignore_eos`)."""
    from xyntetik_runner_b200.engine.runner import Runner
    folder = folders["B", "float32"]
    prompts = [traces.random_tokens(60 + i, n, 387) for i, n in enumerate((7, 19, 3, 12))]
    lengths = [25, 9, 31, 17]

    def run(ahead, stop):
        r = Runner(folder, dtype="float32", ctx=128, parallel=4, page_size=8)
        r.scheduler.params.look_ahead = ahead
        ids = [r.submit(p, n=n, temp=temp, seed=5 + i, stop_ids=stop if i == 2 else (frequent if i == 3 else []),
                        ignore_eos=i == 3, repeat_penalty=penalty)
               for i, (p, n) in enumerate(zip(prompts, lengths))]
        while r.scheduler.has_work():
            r.scheduler.step()
        r.engine.cache.audit()
        assert not r.engine.cache.live_requests()
        done = [r.scheduler.finished[i] for i in ids]
        return [q.generated for q in done], [q.finish_reason for q in done], r.scheduler.stats["steps_launched_ahead"]

    frequent = []
    free, _, n_ahead = run(False, [])
    assert n_ahead == 0 and [len(g) for g in free] == lengths
    frequent = sorted(set(free[3]))[:5]                 # ids that the last request emits: exempt from its penalty from now on
    stop = [free[2][10]]
    want, reasons, _ = run(False, stop)
    assert reasons[2] == "stop" and want[2] == free[2][:free[2].index(stop[0])]
    got, reasons_ahead, n_ahead = run(True, stop)
    assert n_ahead >= 10
    assert got == want and reasons_ahead == reasons


_DIGEST_SCRIPT = """
import hashlib, sys
import numpy as np
sys.path.insert(0, {root!r})
from xyntetik_runner_b200.config.llama import LlamaConfig
from xyntetik_runner_b200.engine.runner import Runner
cfg = LlamaConfig.from_dict({{"architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "num_hidden_layers": 2,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336, "vocab_size": 32000,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "max_position_embeddings": 2048, "tie_word_embeddings": False,
    "hidden_act": "silu", "torch_dtype": "bfloat16"}})
rng = np.random.RandomState(1)
prompts = [[int(t) for t in rng.randint(0, cfg.vocab_size, size=n)] for n in (700, 333, 64, 17, 450, 1100)]
r = Runner(config=cfg, random_seed=5, ctx=2048, batch=1024, parallel=6)
h = hashlib.sha256()
for g in r.generate(prompts, n=48, ignore_eos=True):
    h.update(np.asarray(g.tokens, dtype=np.int64).tobytes())
print("digest", h.hexdigest(), r.engine.graph_replays)
"""


def test_dependent_launch_and_copy_variants_change_no_token(tmp_path):
    """Kernels start before the kernel ahead of them has ended and read, until they wait, only what a step does not
    change (weights, the step's description, keys of earlier steps).  If one read anything else early, tokens
    would depend on timing: the same greedy run at 8B layer sizes must give the same ids with programmatic
    dependent launch switched off, and with the decode attention's bulk copies replaced by per-thread copies
    (compared where the spans are combined by the merge kernel in both: the cluster's exchange adds in another order)."""
    script = tmp_path / "digest.py"
    script.write_text(_DIGEST_SCRIPT.format(root=ROOT))
    digests = []
    for extra in ({}, {"XRB200_NO_PDL": "1"}, {"XRB200_NO_CLUSTER_MERGE": "1"},
                  {"XRB200_NO_CLUSTER_MERGE": "1", "XRB200_NO_TMA_ATTENTION": "1"}):
        p = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, env=dict(os.environ, **extra), timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        line = [l for l in p.stdout.splitlines() if l.startswith("digest")][-1].split()
        assert int(line[2]) > 20                     # decode steps were replayed from CUDA graphs
        digests.append(line[1])
    assert digests[0] == digests[1] and digests[2] == digests[3]


def test_starved_pool_preempts_and_gives_the_same_tokens(folders):
    from xyntetik_runner_b200.engine.runner import Runner
    folder = folders["A", "float32"]
    prompts = [traces.random_tokens(40 + i, n, 256) for i, n in enumerate((30, 22, 27, 18))]
    ample = Runner(folder, dtype="float32", ctx=128, parallel=4, page_size=8)
    want = [g.tokens for g in ample.generate(prompts, n=40, temp=0.0, ignore_eos=True)]
    tight = Runner(folder, dtype="float32", ctx=128, parallel=4, page_size=8, max_tokens=20 * 8)
    got = tight.generate(prompts, n=40, temp=0.0, ignore_eos=True)
    assert tight.scheduler.stats["preemptions"] >= 1
    assert [g.tokens for g in got] == want
    tight.engine.cache.audit()
    assert tight.engine.cache.free_pages() == [20]


def test_command_line(folders, tmp_path):
    folder = folders["A", "float32"]
    plain = PlainLlama(folder)
    ids = [65, 66, 67, 68, 69]
    want = plain.generate_greedy([1] + ids, 6)          # BOS (id 1) is prepended
    env = dict(os.environ, PYTHONPATH=ROOT)
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "runner"), "-m", folder, "-p", "ABCDE", "-n", "6",
                          "--temp", "0", "--ignore-eos", "--dtype", "float32", "-c", "64"],
                         capture_output=True, env=env, timeout=300)
    assert out.returncode == 0, out.stderr.decode(errors="replace")
    lines = out.stdout.split(b"\n")
    assert lines[0].decode() == "ids:" + ",".join(map(str, want))
    assert lines[1] == bytes(want)              # every id is a byte here, so the bytes are printed too
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "runner"), "-m", folder, "-p", "ids:3,4", "-s", "0",
                          "--temp", "0.5"], capture_output=True, text=True, env=env, timeout=300)
    assert out.returncode == 2 and "refused" in out.stderr


def test_context_fitted_to_memory_and_batched_bench_json(folders):
    """-c 0 (the reference's auto-fit): the context is the model's limit when memory allows; --bench-json with
    --parallel runs that many 512-token prompts at once and reports the phases' rates with a per-kernel table."""
    from xyntetik_runner_b200.cli import main
    from xyntetik_runner_b200.engine.runner import Runner
    folder = folders["A", "bfloat16"]
    r = Runner(folder, ctx=0, parallel=2, page_size=16)
    assert r.engine.cache.max_pages_per_request * 16 == 1024        # tiny A's max_position_embeddings
    del r
    import contextlib
    import io
    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        assert main(["-m", folder, "--bench-json", "-n", "12", "--parallel", "3", "-c", "0", "--page-size", "16"]) == 0
    d = json.loads(buf.getvalue().strip().splitlines()[-1])
    assert d["batch"] == 3 and d["prompt_tokens"] == 3 * 512 and d["gen_tokens"] == 36 and d["gen_tok_s"] > 0 and d["prompt_tok_s"] > 0
    names = [row["kernel"] for row in d["kernels"]]
    assert any("attention" in n for n in names) and any("head product" in n for n in names)
    assert all(row["us"] > 0 and 0 <= row["frac"] < 1.5 for row in d["kernels"])      # (a tiny model: fractions near zero)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_scoring(folders, dtype):
    """Runner.score (the reference's --score): per-token log-probabilities of a prompt, whatever the portion."""
    from plain_llama import score_logprobs
    from xyntetik_runner_b200 import Runner
    folder = folders["B", dtype]
    toks = traces.random_tokens(31, 90, tiny.CONFIGS["B"]["vocab_size"])
    plain_logits = PlainLlama(folder).logits(toks)
    want = score_logprobs(plain_logits, toks)
    r = Runner(folder, dtype=dtype, ctx=128, parallel=1, page_size=8)
    # a log-probability is a logit minus a soft maximum of logits: twice the logits' own tolerance
    tol = 2 * traces.TOL[dtype]["max_rel"] * float(np.abs(plain_logits).max())
    for portion in (256, 7, 1):
        got = np.array(r.score(toks, portion=portion), dtype=np.float32)
        assert got.shape == want.shape and np.isfinite(got).all()
        assert np.abs(got - want).max() <= tol, (portion, float(np.abs(got - want).max()))
    assert not r.engine.cache.live_requests()
    with pytest.raises(ValueError, match="at least 2 tokens"):
        r.score([5])


def test_rope_base_override(folders, tmp_path):
    """Runner(rope_base=...) (the command line's --rope-base) is the model whose config.json names that base."""
    import shutil
    from xyntetik_runner_b200 import Runner
    src = folders["A", "float32"]
    dst = str(tmp_path / "other_base")
    shutil.copytree(src, dst)
    with open(os.path.join(dst, "config.json")) as f:
        cfg = json.load(f)
    cfg["rope_theta"] = 777.0
    with open(os.path.join(dst, "config.json"), "w") as f:
        json.dump(cfg, f)
    toks = traces.random_tokens(5, 40, tiny.CONFIGS["A"]["vocab_size"])
    a = Runner(src, dtype="float32", ctx=64, rope_base=777.0).score(toks)
    b = Runner(dst, dtype="float32", ctx=64).score(toks)
    c = Runner(src, dtype="float32", ctx=64).score(toks)
    assert a == b and a != c
    # --rope-scale: forced linear scaling is the model whose config.json asks for it, and the plain implementation's
    from plain_llama import score_logprobs
    cfg["rope_theta"] = tiny.CONFIGS["A"]["rope_theta"]
    cfg["rope_scaling"] = {"rope_type": "linear", "factor": 3.0}
    with open(os.path.join(dst, "config.json"), "w") as f:
        json.dump(cfg, f)
    d = Runner(src, dtype="float32", ctx=64, rope_scale=3.0).score(toks)
    e = Runner(dst, dtype="float32", ctx=64).score(toks)
    plain_logits = PlainLlama(dst).logits(toks)
    tol = 2 * traces.TOL["float32"]["max_rel"] * float(np.abs(plain_logits).max())
    assert d == e and d != c and np.abs(np.array(e) - score_logprobs(plain_logits, toks)).max() <= tol


def test_command_line_scoring(folders):
    from plain_llama import score_logprobs
    folder = folders["A", "float32"]
    ids = [1, 65, 66, 67, 68, 69, 70]
    plain_logits = PlainLlama(folder).logits(ids)
    want = score_logprobs(plain_logits, ids)
    tol = 2 * traces.TOL["float32"]["max_rel"] * float(np.abs(plain_logits).max())
    env = dict(os.environ, PYTHONPATH=ROOT)
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "runner"), "-m", folder, "-p", "ABCDEF", "--score",
                          "--dtype", "float32", "-c", "64"], capture_output=True, text=True, env=env, timeout=300)
    assert out.returncode == 0, out.stderr
    d = json.loads(out.stdout)
    assert d["schema_version"] == "xyntetik.runner.score.v1" and d["tokens"] == ids and d["n_scored"] == 6
    assert np.abs(np.array(d["logprobs"]) - want).max() <= tol
    assert abs(d["nll_total"] + float(want.astype(np.float64).sum())) <= 6 * tol and abs(d["ppl"] - np.exp(d["nll_mean"])) <= 1e-4


def test_trace_run_program(folders, tmp_path):
    """bin/trace_run as a user runs it: steps on standard input, <step>.f32 files and `done` lines out."""
    folder = folders["B", "bfloat16"]
    reqs = {"a": traces.random_tokens(1, 45, 387), "b": traces.random_tokens(2, 70, 387)}
    steps = traces.mixed(reqs, seed=5, max_live=2)
    out_dir = tmp_path / "out"
    env = dict(os.environ, PYTHONPATH="")
    p = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "bfloat16", "--out",
                        str(out_dir), "--max-tokens", str(traces.pool_tokens(steps))],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, env=env,
                       timeout=300)
    assert p.returncode == 0, p.stderr
    assert p.stdout.split() == [w for s in steps for w in ("done", str(s["step"]))]
    res = {s["step"]: np.fromfile(out_dir / f"{s['step']}.f32", dtype="<f4") for s in steps}
    got = traces.collect(steps, res, 387)
    plain = PlainLlama(folder)
    for rid, toks in reqs.items():
        traces.assert_close(got[rid], plain.logits(toks), "bfloat16", f"trace_run/{rid}")
