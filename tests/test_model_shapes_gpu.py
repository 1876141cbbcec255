"""Layer sizes of the models the benchmarks name, against the plain implementation, in every cutting.

Two layers of each shape with seeded random bfloat16 weights (the 8B shape with its vocabulary cut from 128,256 to
32,000 so that the plain implementation's float64 head stays small; the 1B shape keeps the full, tied vocabulary).
The weights exist nowhere on disk: the engine draws them on the device and the plain implementation is handed the
same values, because element i of a tensor is a function of (seed, name, i) alone (weights/random_fill.py).
Both engine paths -- the serving kernels (tcgen05 products on packed weights, tcgen05 prompt attention, bulk-copy
decode attention at head sizes 128 and 64) and the true 32-bit path -- are compared with the plain logits at
the ends of every portion: whole, tail decoded one by one, portions of changing size, mixed; and requests long
enough that decoding crosses a context bucket of the step graphs (1,024) and the span count of the decode
attention changes under test.  The reference compares its device path with its CPU model the same way
(tests/test_gpu_identity.c:60-108)."""
import numpy as np
import pytest
import torch

import traces
from plain_llama import PlainLlama

pytestmark = pytest.mark.gpu

SHAPE_8B = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "num_hidden_layers": 2, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336, "vocab_size": 32000, "rms_norm_eps": 1e-5,
    "rope_theta": 500000.0, "rope_scaling": None, "max_position_embeddings": 8192, "tie_word_embeddings": False,
    "hidden_act": "silu", "torch_dtype": "bfloat16",
}
# Llama-3.2-1B layer sizes: head size 64, tied head over the full vocabulary, llama3 rope scaling x32
SHAPE_1B = dict(SHAPE_8B, hidden_size=2048, head_dim=64, intermediate_size=8192, vocab_size=128256, tie_word_embeddings=True,
                rope_scaling={"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                              "original_max_position_embeddings": 8192})
# Llama-2-13B layer sizes: as many kv heads as heads, theta 10000
SHAPE_13B = dict(SHAPE_8B, hidden_size=5120, num_attention_heads=40, num_key_value_heads=40, intermediate_size=13824,
                 rope_theta=10000.0, max_position_embeddings=4096)
SHAPES = {"llama-3-8b": (SHAPE_8B, 2), "llama-3.2-1b": (SHAPE_1B, 3), "llama-2-13b": (SHAPE_13B, 4)}
STD = 0.02


def only_ends(steps, keep=2):
    """ask for logits at the last `keep` tokens of every entry only (a row of logits is up to half a megabyte)"""
    for st in steps:
        for e in st["entries"]:
            e["want"] = list(range(max(0, len(e["tokens"]) - keep), len(e["tokens"])))
    return steps


def long_requests(reqs):
    """Prefill in one step or in uneven portions, then single tokens: decoding crosses position 1,024 (a new context
    bucket, so a new step graph and another span count of the decode attention)."""
    steps, k = [], 0
    for rid, (toks, head, sizes) in reqs.items():
        at, j = 0, 0
        while at < head:
            m = min(sizes[j % len(sizes)], head - at)
            steps.append({"step": k, "entries": [{"id": rid, "tokens": toks[at:at + m]}], "end": []})
            at, j, k = at + m, j + 1, k + 1
        for i in range(head, len(toks)):
            steps.append({"step": k, "entries": [{"id": rid, "tokens": [toks[i]]}], "end": [rid] if i == len(toks) - 1 else []})
            k += 1
    return only_ends(steps, keep=1)


def rows_of(steps, results):
    """{(request, position): logits row} of a replay."""
    out, at_of = {}, {}
    for st in steps:
        arr, at = results.get(st["step"]), 0
        for e in st["entries"]:
            p0 = at_of.get(e["id"], 0)
            for w in e["want"]:
                out[e["id"], p0 + w] = arr[at]
                at += 1
            at_of[e["id"]] = p0 + len(e["tokens"])
    return out


@pytest.fixture(scope="module", params=list(SHAPES))
def shape_case(request):
    """(name, typed configuration, requests, traces by cutting, plain logits at every wanted place)."""
    from xyntetik_runner_b200.architectures.llama import build_llama
    from xyntetik_runner_b200.config.llama import LlamaConfig
    from xyntetik_runner_b200.weights.loader import RandomSource
    name = request.param
    shape, seed = SHAPES[name]
    cfg = LlamaConfig.from_dict(shape)
    V = cfg.vocab_size
    reqs = {"a": traces.random_tokens(1, 150, V), "b": traces.random_tokens(2, 70, V),
            "c": traces.random_tokens(3, 600, V)}          # 600: several token tiles of the CTA-pair product
    cuts = {"whole": only_ends(traces.whole(reqs)), "tail": only_ends(traces.tail_decoded(reqs, 32)),
            "portions": only_ends(traces.portions(reqs, sizes=(97, 3, 2, 130, 2, 45, 1, 17, 260, 4))),
            "mixed": only_ends(traces.mixed(reqs, seed=4, max_live=3, sizes=(1, 1, 2, 50, 1, 9, 130, 1, 16, 2)))}
    if name != "llama-2-13b":
        # d: one step to position 1,000, then 60 tokens one by one; e (head size 64 only: the plain side's cost):
        # uneven portions to 2,030, then 40 tokens one by one across 2,048
        longs = {"d": (traces.random_tokens(5, 1060, V), 1000, (1000,))}
        if name == "llama-3.2-1b":
            longs["e"] = (traces.random_tokens(6, 2070, V), 2030, (515, 2, 700, 130, 3))
        cuts["long"] = long_requests(longs)
        reqs = dict(reqs, **{rid: t[0] for rid, t in longs.items()})
    # the plain side: the same values the engine will draw, tensor by tensor
    src = RandomSource(build_llama(cfg).tensor_specs(), seed, torch.bfloat16, std=STD, norm_jitter=0.1, gen_device="cuda:0")
    tensors = {n: src.fetch(n, torch.device("cuda:0")).float().cpu().numpy() for n in src.specs}
    plain = PlainLlama(config=shape, tensors=tensors)
    wanted = {}
    for steps in cuts.values():
        at_of = {}
        for st in steps:
            for e in st["entries"]:
                p0 = at_of.get(e["id"], 0)
                wanted.setdefault(e["id"], set()).update(p0 + w for w in e["want"])
                at_of[e["id"]] = p0 + len(e["tokens"])
    ref = {}
    for rid, toks in reqs.items():
        rows = sorted(wanted[rid])
        lg = plain.logits(toks, rows=rows)
        for r, row in zip(rows, lg):
            ref[rid, r] = row
    del plain, tensors
    return name, cfg, seed, cuts, ref


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_cutting_matches_plain_at_benchmark_layer_sizes(shape_case, dtype):
    from xyntetik_runner_b200.engine.engine import EngineParams, random_engine
    from xyntetik_runner_b200.engine.replay import replay
    from xyntetik_runner_b200.parts import attention, linear
    name, cfg, seed, cuts, ref = shape_case
    pool = max(traces.pool_tokens(steps) for steps in cuts.values())
    eng = random_engine(cfg, seed, EngineParams(dtype=dtype, max_tokens=pool, page_size=64, max_requests=3, max_step_tokens=1024),
                        std=STD, norm_jitter=0.1)
    before, before_att = dict(linear.counters), dict(attention.counters)
    tol = traces.TOL[dtype]
    compared = 0
    for cut_name, steps in cuts.items():
        replays0 = eng.graph_replays
        res = replay(eng, steps)
        eng.cache.audit()
        assert not eng.cache.live_requests()
        got = rows_of(steps, res)
        worst = (0.0, None)
        for key, row in got.items():
            want = ref[key]
            scale = float(np.abs(want).max())
            d = np.abs(row.astype(np.float64) - want)
            assert np.isfinite(row).all(), (name, cut_name, key)
            if d.max() / scale > worst[0]:
                worst = (d.max() / scale, key)
            assert d.max() <= tol["max_rel"] * scale and d.mean() <= tol["mean_rel"] * scale, \
                f"{name}/{cut_name}/{dtype}: request {key[0]} position {key[1]}: max {d.max() / scale:.2e} mean {d.mean() / scale:.2e}"
            compared += 1
        if cut_name == "long":
            assert eng.graph_replays - replays0 >= 40          # the single-token steps ran as replayed graphs, new bucket included
            assert len({k[2] for k in eng._graph_seen}) >= 2    # in two context buckets
    assert compared > 150
    used_tc = linear.counters["tcgen05"] - before["tcgen05"]
    assert (used_tc > 0) == (dtype == "bfloat16")              # the tensor-core product ran iff serving path
    if dtype == "bfloat16":
        assert attention.counters["tcgen05"] > before_att["tcgen05"] and attention.counters["mma"] > before_att["mma"]
    del eng
    torch.cuda.empty_cache()


def test_32_bit_path_gives_the_same_bits_in_every_cutting(shape_case):
    """The true 32-bit path at these sizes: a position's logits are bit-identical however the work was cut."""
    from xyntetik_runner_b200.engine.engine import EngineParams, random_engine
    from xyntetik_runner_b200.engine.replay import replay
    name, cfg, seed, cuts, ref = shape_case
    small = {k: v for k, v in cuts.items() if k != "long"}
    pool = max(traces.pool_tokens(steps) for steps in small.values())
    eng = random_engine(cfg, seed, EngineParams(dtype="float32", max_tokens=pool, page_size=64, max_requests=3, max_step_tokens=1024),
                        std=STD, norm_jitter=0.1)
    rows = {c: rows_of(steps, replay(eng, steps)) for c, steps in small.items()}
    common = 0
    for c in ("tail", "portions", "mixed"):
        for key, row in rows[c].items():
            if key in rows["whole"]:
                assert np.array_equal(row, rows["whole"][key]), (name, c, key)
                common += 1
    assert common >= 9
    del eng
    torch.cuda.empty_cache()


def test_device_and_host_draw_the_same_weights():
    """The generator's CUDA kernel and its numpy twin: the same bits, whole tensors and pieces of a large one, in
    float32 and rounded to bfloat16."""
    from xyntetik_runner_b200 import kernels
    from xyntetik_runner_b200.weights import random_fill as rf
    dev = torch.device("cuda:0")
    for seed, name, n, mean, std in ((0, "a.weight", 1, 0.0, 0.02), (2, "model.embed_tokens.weight", 100003, 0.0, 0.02),
                                     (3, "norm", 4097, 1.0, 0.1), (9, "x", 1 << 21, -0.5, 3.0)):
        key = rf.tensor_key(seed, name)
        host = rf.normal_values(key, 0, n, mean, std)
        for dt in (torch.float32, torch.bfloat16):
            out = torch.empty(n, dtype=dt, device=dev)
            kernels.random_normal(out, key, mean, std)
            if dt == torch.float32:
                assert np.array_equal(out.cpu().numpy().view(np.uint32), host.view(np.uint32)), (name, "float32")
            else:
                assert np.array_equal(out.view(torch.int16).cpu().numpy().view(np.uint16), rf.to_bfloat16_bits(host)), (name, "bfloat16")
    # a slice far into a tensor of 2^33 elements: the index is 64 bits wide on both sides
    key = rf.tensor_key(1, "big")
    first = (1 << 33) + 12345
    out = torch.empty(5000, dtype=torch.float32, device=dev)
    kernels.random_normal(out, key, 0.0, 1.0, first=first)
    assert np.array_equal(out.cpu().numpy(), rf.normal_values(key, first, 5000, 0.0, 1.0))
    z = rf.normal_values(key, 0, 1 << 20, 0.0, 1.0)
    assert abs(float(z.mean())) < 5e-3 and abs(float(z.std()) - 1.0) < 5e-3 and abs(float((z ** 4).mean()) - 3.0) < 0.05


MANY = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 512, "num_hidden_layers": 2, "num_attention_heads": 16,
    "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 1024, "vocab_size": 1000, "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0, "rope_scaling": None, "max_position_embeddings": 2048, "tie_word_embeddings": False,
    "hidden_act": "silu", "torch_dtype": "bfloat16",
}


@pytest.mark.parametrize("n_requests", [48, 14])
def test_many_requests_of_unequal_length_decode_together(n_requests):
    """48 requests x 8 kv heads are more (request, kv head) pairs than CTAs of the decode attention fit on the machine,
    and 14 requests of 5 to 1,300 tokens are few but uneven: both go through the kernel that cuts the tiles of all
    requests into even shares.  Prompts of 5 to 1,300 tokens, then six tokens each decoded together (plainly, captured,
    replayed), every decoded position against the plain implementation."""
    from xyntetik_runner_b200 import kernels
    from xyntetik_runner_b200.architectures.llama import build_llama
    from xyntetik_runner_b200.config.llama import LlamaConfig
    from xyntetik_runner_b200.engine.engine import EngineParams, random_engine
    from xyntetik_runner_b200.engine.replay import replay
    from xyntetik_runner_b200.weights.loader import RandomSource
    cfg = LlamaConfig.from_dict(MANY)
    seed, V, n_decoded = 11, cfg.vocab_size, 6
    rng = np.random.RandomState(n_requests)
    lengths = [5, 63, 64, 65, 1300] + [int(x) for x in rng.randint(20, 1100, size=n_requests - 5)]
    reqs = {f"r{i}": traces.random_tokens(100 + i, n + n_decoded, V) for i, n in enumerate(lengths)}
    steps, batch, room = [], [], 2048
    for rid, toks in reqs.items():
        n = len(toks) - n_decoded
        if n > room:
            steps.append({"step": len(steps), "entries": batch, "end": []})
            batch, room = [], 2048
        batch.append({"id": rid, "tokens": toks[:n], "want": []})
        room -= n
    steps.append({"step": len(steps), "entries": batch, "end": []})
    for j in range(n_decoded):
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [toks[len(toks) - n_decoded + j]], "want": [0]}
                                                      for rid, toks in reqs.items()],
                      "end": list(reqs) if j == n_decoded - 1 else []})
    src = RandomSource(build_llama(cfg).tensor_specs(), seed, torch.bfloat16, std=0.05, norm_jitter=0.1, gen_device="cuda:0")
    tensors = {n: src.fetch(n, torch.device("cuda:0")).float().cpu().numpy() for n in src.specs}
    plain = PlainLlama(config=MANY, tensors=tensors)
    eng = random_engine(cfg, seed, EngineParams(dtype="bfloat16", max_tokens=traces.pool_tokens(steps), page_size=64,
                                                max_requests=n_requests, max_step_tokens=2048), std=0.05, norm_jitter=0.1)
    even0 = kernels.attention_even_launches()
    res = replay(eng, steps)
    eng.cache.audit()
    assert kernels.attention_even_launches() >= even0 + 2 * cfg.num_hidden_layers      # the plain decode step and the captured one
    assert eng.graph_replays >= n_decoded - 2
    assert int(kernels.workspace(torch.device("cuda:0")).flags.abs().sum()) == 0
    tol = traces.TOL["bfloat16"]
    first = len(steps) - n_decoded
    for i, (rid, toks) in enumerate(reqs.items()):
        rows = list(range(len(toks) - n_decoded, len(toks)))
        want = plain.logits(toks, rows=rows)
        for j, w in enumerate(want):
            row = res[first + j][i]
            scale = float(np.abs(w).max())
            d = np.abs(row.astype(np.float64) - w)
            assert np.isfinite(row).all() and d.max() <= tol["max_rel"] * scale and d.mean() <= tol["mean_rel"] * scale, \
                f"request {rid} ({len(toks) - n_decoded} tokens), decoded token {j}: max {d.max() / scale:.2e} mean {d.mean() / scale:.2e}"
    del eng
    torch.cuda.empty_cache()


LONG = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 128, "num_hidden_layers": 2, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 320, "vocab_size": 300, "rms_norm_eps": 1e-5,
    "rope_theta": 500000.0, "max_position_embeddings": 16384, "tie_word_embeddings": False, "hidden_act": "silu",
    "torch_dtype": "bfloat16",
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 2048},
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_across_position_8192(dtype):
    """The benchmark's context length, checked: a prompt of 8,150 tokens in portions of 2,048 (the last portions attend
    to thousands of cached keys), then 80 tokens decoded one by one beside a request of a few hundred tokens, across
    position 8,192 (a new context bucket of the step graphs, 129 pages of 64, rotation angles of thousands of radians in
    float32).  Every decoded position and the last prompt position against the plain implementation."""
    from xyntetik_runner_b200.architectures.llama import build_llama
    from xyntetik_runner_b200.config.llama import LlamaConfig
    from xyntetik_runner_b200.engine.engine import EngineParams, random_engine
    from xyntetik_runner_b200.engine.replay import replay
    from xyntetik_runner_b200.weights.loader import RandomSource
    cfg = LlamaConfig.from_dict(LONG)
    seed, V, head, n_decoded = 21, cfg.vocab_size, 8150, 80
    reqs = {"long": traces.random_tokens(7, head + n_decoded, V), "short": traces.random_tokens(8, 300 + n_decoded, V)}
    steps = []
    for at in range(0, head, 2048):
        m = min(2048, head - at)
        steps.append({"step": len(steps), "entries": [{"id": "long", "tokens": reqs["long"][at:at + m], "want": [m - 1] if at + m == head else []}], "end": []})
    steps.append({"step": len(steps), "entries": [{"id": "short", "tokens": reqs["short"][:300], "want": [299]}], "end": []})
    for j in range(n_decoded):
        steps.append({"step": len(steps), "entries": [{"id": "long", "tokens": [reqs["long"][head + j]], "want": [0]},
                                                      {"id": "short", "tokens": [reqs["short"][300 + j]], "want": [0]}],
                      "end": ["long", "short"] if j == n_decoded - 1 else []})
    src = RandomSource(build_llama(cfg).tensor_specs(), seed, torch.bfloat16, std=0.08, norm_jitter=0.1, gen_device="cuda:0")
    tensors = {n: src.fetch(n, torch.device("cuda:0")).float().cpu().numpy() for n in src.specs}
    plain = PlainLlama(config=LONG, tensors=tensors)
    eng = random_engine(cfg, seed, EngineParams(dtype=dtype, max_tokens=traces.pool_tokens(steps), page_size=64, max_requests=2,
                                                max_step_tokens=2048), std=0.08, norm_jitter=0.1)
    res = replay(eng, steps)
    eng.cache.audit()
    assert eng.graph_replays >= n_decoded - 6 and len({k[2] for k in eng._graph_seen}) == 2      # two context buckets
    ref = {"long": plain.logits(reqs["long"], rows=list(range(head - 1, head + n_decoded))),
           "short": plain.logits(reqs["short"], rows=list(range(299, 300 + n_decoded)))}
    first = len(steps) - n_decoded
    got = {"long": [res[first - 2][0]] + [res[first + j][0] for j in range(n_decoded)],
           "short": [res[first - 1][0]] + [res[first + j][1] for j in range(n_decoded)]}
    tol = traces.TOL[dtype]
    for rid in reqs:
        for j, (row, want) in enumerate(zip(got[rid], ref[rid])):
            scale = float(np.abs(want).max())
            d = np.abs(row.astype(np.float64) - want)
            assert np.isfinite(row).all() and d.max() <= tol["max_rel"] * scale and d.mean() <= tol["mean_rel"] * scale, \
                f"{dtype}: request {rid}, row {j} of {n_decoded + 1}: max {d.max() / scale:.2e} mean {d.mean() / scale:.2e}"
    del eng
    torch.cuda.empty_cache()
