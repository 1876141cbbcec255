"""Replay of the same requests cut in every way, in 32 bit and in bfloat16, against the plain implementation."""
import numpy as np
import pytest

import tiny
import traces
from plain_llama import PlainLlama

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 11, 17, 70, 130, 41], "B": [1, 9, 33, 70, 150, 64], "C": [3, 29, 66, 100, 129, 48],
           "D": [2, 19, 90, 35, 60, 77, 50, 88], "E": [7, 140, 33, 64, 90, 21]}
PAGE = {"A": 16, "B": 8, "C": 64, "D": 4, "E": 32}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name in "ABCDE":
        for dt in ("float32", "bfloat16"):
            out[name, dt] = tiny.make_folder(str(tmp_path_factory.mktemp(f"tiny{name}_{dt}")), name, dt)
    return out


@pytest.fixture(scope="module")
def reference(folders):
    """Plain logits of every request, per (config, weight dtype)."""
    out = {}
    for (name, dt), folder in folders.items():
        vocab = tiny.CONFIGS[name]["vocab_size"]
        reqs = {f"r{i}": traces.random_tokens(100 * i + ord(name), n, vocab) for i, n in enumerate(LENGTHS[name])}
        m = PlainLlama(folder)
        out[name, dt] = (reqs, {rid: m.logits(t) for rid, t in reqs.items()})
    return out


def run(folder, dtype, steps, page_size, max_tokens=None, max_requests=4):
    from xyntetik_runner_b200.engine.engine import Engine, EngineParams
    from xyntetik_runner_b200.engine.replay import replay
    mt = max_tokens if max_tokens is not None else traces.pool_tokens(steps)
    eng = Engine(folder, EngineParams(dtype=dtype, max_tokens=mt, page_size=page_size, max_requests=max_requests))
    res = replay(eng, steps)
    eng.cache.audit()
    assert not eng.cache.live_requests()
    return res, eng


CUTS = {
    "whole": lambda reqs: traces.whole(reqs),
    "tail": lambda reqs: traces.tail_decoded(reqs, 32),
    "portions": lambda reqs: traces.portions(reqs),
    "mixed": lambda reqs: traces.mixed(reqs, seed=3),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cut", list(CUTS))
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_cutting_matches_plain(folders, reference, name, cut, dtype):
    reqs, ref = reference[name, dtype]
    steps = CUTS[cut](reqs)
    res, eng = run(folders[name, dtype], dtype, steps, PAGE[name])
    got = traces.collect(steps, res, tiny.CONFIGS[name]["vocab_size"])
    for rid in reqs:
        traces.assert_close(got[rid], ref[rid], dtype, f"{name}/{cut}/{dtype}/{rid}")
    if cut == "mixed":
        # the pool was sized for the peak, so pages of finished requests were used again
        total = sum(-(-len(t) // PAGE[name]) for t in reqs.values())
        assert total > eng.cache.pools[0].n_pages


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(folders, dtype):
    """40 tokens at once, then 260 tokens one by one (pages fill and new ones are taken many times)."""
    name = "A"
    toks = traces.random_tokens(77, 300, tiny.CONFIGS[name]["vocab_size"])
    ref = PlainLlama(folders[name, dtype]).logits(toks)
    steps = traces.tail_decoded({"long": toks}, tail=260)
    res, eng = run(folders[name, dtype], dtype, steps, page_size=16, max_tokens=320)
    got = traces.collect(steps, res, tiny.CONFIGS[name]["vocab_size"])["long"]
    traces.assert_close(got, ref, dtype, f"long decoding/{dtype}")
    if dtype == "bfloat16":
        assert eng.graph_replays > 200          # the decode steps ran as replayed graphs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_first_tokens(folders, name, dtype):
    """Positions 0, 1, 2 of a sequence: whole, and token by token from the very first."""
    vocab = tiny.CONFIGS[name]["vocab_size"]
    plain = PlainLlama(folders[name, dtype])
    reqs = {f"f{n}": traces.random_tokens(n, n, vocab) for n in (1, 2, 3)}
    for cut in (traces.whole, lambda r: traces.tail_decoded(r, tail=8)):
        steps = cut(reqs)
        res, _ = run(folders[name, dtype], dtype, steps, PAGE[name])
        got = traces.collect(steps, res, vocab)
        for rid, t in reqs.items():
            traces.assert_close(got[rid], plain.logits(t), dtype, f"first tokens/{name}/{rid}")


def test_batch_does_not_change_a_request_in_32_bit(folders):
    """float32 path: a request's logits are bit-identical alone, in portions, and mixed with others."""
    name = "B"
    vocab = tiny.CONFIGS[name]["vocab_size"]
    reqs = {f"r{i}": traces.random_tokens(50 + i, n, vocab) for i, n in enumerate((40, 75, 23, 61))}
    outs = []
    for cut in (traces.whole, traces.portions, lambda r: traces.mixed(r, seed=9)):
        steps = cut(reqs)
        res, _ = run(folders[name, "float32"], "float32", steps, 8)
        outs.append(traces.collect(steps, res, vocab))
    for rid in reqs:
        assert np.array_equal(outs[0][rid], outs[1][rid]) and np.array_equal(outs[0][rid], outs[2][rid]), rid


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_batches_of_shrinking_size(folders, dtype):
    """Thirteen requests decode together and end one after another.  Decode-only steps of more than eight requests
    are filled up to a multiple of eight with rows of no request, so that the sizes of the steps repeat and their
    CUDA graphs are few; the logits of the real rows are those of the plain implementation, and a request that
    shares a step with filler rows is not changed by them."""
    name = "B"
    vocab = tiny.CONFIGS[name]["vocab_size"]
    plain = PlainLlama(folders[name, dtype])
    reqs = {f"q{i}": traces.random_tokens(900 + i, 18 + 3 * i, vocab) for i in range(13)}
    tail = {rid: 4 + 2 * i for i, rid in enumerate(reqs)}                    # tokens decoded one by one, all different
    steps, k = [], 0
    for rid, toks in reqs.items():
        head = len(toks) - tail[rid]
        steps.append({"step": k, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        k += 1
    at = {rid: len(t) - tail[rid] for rid, t in reqs.items()}
    sizes = []
    while any(at[rid] < len(reqs[rid]) for rid in reqs):
        live = [rid for rid in reqs if at[rid] < len(reqs[rid])]
        entries = [{"id": rid, "tokens": [reqs[rid][at[rid]]], "want": [0]} for rid in live]
        for rid in live:
            at[rid] += 1
        steps.append({"step": k, "entries": entries, "end": [rid for rid in live if at[rid] == len(reqs[rid])]})
        sizes.append(len(live))
        k += 1
    assert max(sizes) == 13 and len(set(sizes)) >= 10                        # the batch really shrinks step by step
    res, eng = run(folders[name, dtype], dtype, steps, PAGE[name], max_requests=16)
    got = traces.collect(steps, res, vocab)
    for rid, toks in reqs.items():
        traces.assert_close(got[rid], plain.logits(toks), dtype, f"shrinking batch/{dtype}/{rid}")
    # sizes 9..13 all ran as steps of 16 rows: one graph for them, replayed
    assert sum(1 for key in eng._graphs if key[0] == 16) <= 1 and not any(8 < key[0] < 16 for key in eng._graph_seen)
    assert eng.graph_replays >= sum(1 for s in sizes if s > 8) - 2
