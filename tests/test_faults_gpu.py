"""Failures injected on the host: a launcher that raises, a pool that refuses.  Nothing here makes the device fail.

The rule under test is the reference's for a position handed out for a forward that never ran ("a step whose forward
never happened owns no KV row: give it back", src/engine.c:1917-1925): after a failed step the cache is as before
the call, the step can be run again, and what other requests compute afterwards is bit for bit what it would have
been without the failure."""
import numpy as np
import pytest

import tiny
import traces

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    return tiny.make_folder(str(tmp_path_factory.mktemp("faultsB")), "B", "float32")


def make_engine(folder, **kw):
    from xyntetik_runner_b200.engine.engine import Engine, EngineParams
    p = dict(dtype="float32", max_tokens=512, page_size=8, max_requests=4, cuda_graphs=False)
    p.update(kw)
    return Engine(folder, EngineParams(**p))


def fail_on_call(monkeypatch, name, nth):
    """kernels.<name> raises KernelError on its nth call from now on (1-based), once."""
    from xyntetik_runner_b200 import kernels
    real = getattr(kernels, name)
    state = {"calls": 0, "raised": 0}

    def wrapper(*a, **k):
        state["calls"] += 1
        if state["calls"] == nth:
            state["raised"] += 1
            raise kernels.KernelError(f"injected: {name} refused its launch")
        return real(*a, **k)
    monkeypatch.setattr(kernels, name, wrapper)
    return state


def snapshot(eng):
    c = eng.cache
    return (c.free_pages(), sorted(map(str, c.live_requests())), {str(r): c.length(r) for r in c.live_requests()},
            [t.copy() for t in c.tables])


def same(a, b):
    return a[0] == b[0] and a[1] == b[1] and a[2] == b[2] and all(np.array_equal(x, y) for x, y in zip(a[3], b[3]))


@pytest.mark.parametrize("launcher,nth", [("embed", 1), ("rmsnorm", 3), ("gemm_simt", 5), ("rope_store", 2), ("attention_simt", 3)])
def test_a_launcher_that_raises_leaves_the_cache_as_before_and_the_step_can_run_again(folder, monkeypatch, launcher, nth):
    from xyntetik_runner_b200 import kernels
    from xyntetik_runner_b200.engine.engine import StepEntry
    V = tiny.TINY_B["vocab_size"]
    toks = {r: traces.random_tokens(i, 40, V) for i, r in enumerate("abc")}
    outs = []
    for inject in (False, True):
        eng = make_engine(folder)
        eng.step([StepEntry("a", toks["a"][:17], [16]), StepEntry("b", toks["b"][:9], [])])
        before = snapshot(eng)
        # a step of three entries: two requests go on, one is new
        entries = [StepEntry("a", toks["a"][17:18], [0]), StepEntry("c", toks["c"][:13], [12]), StepEntry("b", toks["b"][9:20], [10])]
        if inject:
            with monkeypatch.context() as m:
                state = fail_on_call(m, launcher, nth)
                with pytest.raises(kernels.KernelError, match="injected"):
                    eng.step(entries)
                assert state["raised"] == 1
            eng.cache.audit()
            assert same(snapshot(eng), before) and not eng.is_live("c")
            for r in "ab":
                assert eng.cache.reserved(r) == 0
        first = eng.step(entries).cpu().numpy().copy()
        later = eng.step([StepEntry(r, toks[r][eng.length(r):eng.length(r) + 5], [4]) for r in "cab"]).cpu().numpy().copy()
        eng.cache.audit()
        outs.append((first, later, snapshot(eng)))
    assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])
    # (the page numbers may differ: pages that were given back lie in the free list in another order)
    assert outs[0][2][:3] == outs[1][2][:3]


def test_a_pool_that_refuses_the_second_of_three_entries_takes_nothing(folder):
    """All or nothing: the first entry's reservation is undone and the request that the step opened is closed."""
    from xyntetik_runner_b200.cache.pages import OutOfPages
    from xyntetik_runner_b200.engine.engine import StepEntry
    V = tiny.TINY_B["vocab_size"]
    eng = make_engine(folder, max_tokens=64)               # eight pages of eight tokens
    toks = {r: traces.random_tokens(10 + i, 60, V) for i, r in enumerate("abc")}
    eng.step([StepEntry("a", toks["a"][:20], [19])])       # three pages
    before = snapshot(eng)
    entries = [StepEntry("c", toks["c"][:9], [8]),         # two pages: fits
               StepEntry("b", toks["b"][:30], [29]),       # four pages: does not fit beside them
               StepEntry("a", toks["a"][20:21], [0])]
    with pytest.raises(OutOfPages):
        eng.step(entries)
    eng.cache.audit()
    assert same(snapshot(eng), before) and not eng.is_live("c") and not eng.is_live("b")
    # what fits still runs, and gives what a fresh engine gives
    got = eng.step([entries[0], entries[2]]).cpu().numpy().copy()
    fresh = make_engine(folder, max_tokens=64)
    fresh.step([StepEntry("a", toks["a"][:20], [19])])
    assert np.array_equal(got, fresh.step([entries[0], entries[2]]).cpu().numpy())


def test_a_failure_while_a_step_graph_is_captured(folder, monkeypatch):
    """Decode steps are captured as CUDA graphs on their second sighting.  A launcher that raises in the middle of
    the capture ends it; the step is given back like any other, and the next try captures and replays."""
    from xyntetik_runner_b200 import kernels
    from xyntetik_runner_b200.engine.engine import StepEntry
    V = tiny.TINY_B["vocab_size"]
    toks = {r: traces.random_tokens(20 + i, 40, V) for i, r in enumerate("ab")}
    outs = []
    for inject in (False, True):
        eng = make_engine(folder, cuda_graphs=True)
        eng.step([StepEntry("a", toks["a"][:12], []), StepEntry("b", toks["b"][:7], [])])
        rows = []
        for i in range(8):
            entries = [StepEntry("a", [toks["a"][12 + i]], [0]), StepEntry("b", [toks["b"][7 + i]], [0])]
            if inject and i == 1:                          # the second decode step: the capture
                with monkeypatch.context() as m:
                    fail_on_call(m, "gemm_simt", 6)
                    with pytest.raises(kernels.KernelError, match="injected"):
                        eng.step(entries)
                eng.cache.audit()
                assert eng.length("a") == 13 and eng.length("b") == 8
            rows.append(eng.step(entries).cpu().numpy().copy())
        assert eng.graph_replays >= 5
        eng.check_status()
        outs.append(rows)
    for x, y in zip(*outs):
        assert np.array_equal(x, y)


@pytest.mark.parametrize("temp", [0.0, 0.9])
def test_generation_goes_on_after_failed_steps(folder, monkeypatch, temp):
    """Through the scheduler: launchers fail in a prompt step, in a decode step, in a step launched ahead and in the
    sampling that belongs to a step.  The caller sees each exception (but the one of a launch ahead, which is tried
    again in its turn) and goes on stepping; every request ends with the tokens of a run without failures."""
    from xyntetik_runner_b200 import kernels
    from xyntetik_runner_b200.engine.runner import Runner
    V = tiny.TINY_B["vocab_size"]
    prompts = [traces.random_tokens(40 + i, n, V) for i, n in enumerate((5, 30, 17))]
    results = []
    for inject in (False, True):
        r = Runner(folder, dtype="float32", ctx=128, parallel=3, page_size=8, batch=24)
        r.engine._graph_ok = False                         # every step launches its kernels through the patched module
        ids = [r.submit(p, n=14, temp=temp, seed=None if temp == 0 else 5 + i, ignore_eos=True) for i, p in enumerate(prompts)]
        sch = r.scheduler
        plan = {1: ("rmsnorm", 2), 3: ("sample", 1), 4: ("gemm_simt", 9), 7: ("embed", 1), 9: ("sample", 1), 12: ("attention_simt", 2)} if inject else {}
        raised = step_no = 0
        while sch.has_work():
            step_no += 1
            if step_no in plan:
                with monkeypatch.context() as m:
                    state = fail_on_call(m, *plan[step_no])
                    try:
                        sch.step()
                    except kernels.KernelError:
                        raised += 1
                    assert state["raised"] == 1, (step_no, plan[step_no], state)
            else:
                sch.step()
            r.engine.cache.audit()
            assert step_no < 200
        if inject:
            assert raised + sch.stats.get("ahead_launches_failed", 0) == len(plan) and raised >= 2
        assert not r.engine.cache.live_requests()
        results.append([(sch.finished[i].generated, sch.finished[i].finish_reason) for i in ids])
    assert results[0] == results[1]
    assert all(len(g) == 14 for g, _ in results[0])


def test_a_wait_that_runs_out_is_reported_and_the_runner_goes_on(folder):
    """The bounded wait of the decode attention (a piece of a request handed over by another block) on a flag that
    nothing raises: the probe kernel runs that wait for a few thousand looks, it runs out, and the kernel writes the
    status word as the attention kernel would.  Nothing faults or hangs.  The host must then: raise at its next look at
    the word (every `Runner.STATUS_EVERY` steps inside `generate`), clear the word, give back what the call held,
    and generate the same tokens as before when asked again."""
    import torch
    from xyntetik_runner_b200 import kernels
    from xyntetik_runner_b200.engine.runner import Runner
    dev = torch.device("cuda:0")
    kernels.tc_check_status(dev)
    kernels.attention_wait_probe(dev)
    with pytest.raises(kernels.KernelError, match="decode attention gave up waiting"):
        kernels.tc_check_status(dev)
    kernels.tc_check_status(dev)                            # the word was cleared by the look that raised
    ws = kernels.workspace(dev)
    assert int(ws.status.item()) == 0 and int(ws.flags.abs().sum()) == 0

    V = tiny.TINY_B["vocab_size"]
    prompts = [traces.random_tokens(70 + i, n, V) for i, n in enumerate((9, 21, 14))]
    r = Runner(folder, dtype="float32", ctx=128, parallel=3, page_size=8)
    want = [g.tokens for g in r.generate(prompts, n=12, ignore_eos=True)]
    r.STATUS_EVERY = 2
    seen = {"tokens": 0}

    def on_token(rid, tok, done):
        seen["tokens"] += 1
        if seen["tokens"] == 7:
            kernels.attention_wait_probe(dev)               # from here on the status word says that a kernel gave up
        return True
    with pytest.raises(kernels.KernelError, match="gave up waiting"):
        r.generate(prompts, n=12, ignore_eos=True, on_token=on_token)
    assert seen["tokens"] < 3 * 12                          # the call ended at a look at the word, not after all its tokens
    r.engine.cache.audit()
    assert not r.engine.cache.live_requests() and not r.scheduler.has_work() and not r.scheduler.finished
    again = [g.tokens for g in r.generate(prompts, n=12, ignore_eos=True)]
    assert again == want
    r.engine.cache.audit()
