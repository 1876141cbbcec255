"""Replay of the same requests cut in every way, in 32 bit and in bfloat16, against the plain implementation."""
import numpy as np
import pytest

import tiny
import traces
from plain_llama import PlainLlama

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 11, 17, 70, 130, 41], "B": [1, 9, 33, 70, 150, 64], "C": [3, 29, 66, 100, 129, 48]}
PAGE = {"A": 16, "B": 8, "C": 64}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name in "ABC":
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
@pytest.mark.parametrize("name", ["A", "B", "C"])
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
