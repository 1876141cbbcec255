"""The scheduler's decisions, with an executor that computes nothing (no GPU)."""
import numpy as np
import pytest

from xyntetik_runner_b200.cache.pages import CacheManager, GroupSpec
from xyntetik_runner_b200.engine.scheduler import Request, Scheduler, SchedulerParams
from xyntetik_runner_b200.sampling.sampler import RequestSampler, SamplingParams


class FakeExecutor:
    """Commits what was planned and 'samples' a function of (request, position): the token a request gets
    must not depend on batching or preemption."""

    def __init__(self, cache, stop_at=None):
        self.cache, self.plans, self.stop_at = cache, [], stop_at or {}

    def run(self, plan):
        self.plans.append([(e.request.id, e.start, e.count, e.wants_token) for e in plan.entries])
        out = {}
        for e in plan.entries:
            assert self.cache.length(e.request.id) == e.start          # portions are contiguous
            self.cache.commit(e.request.id)
            if e.wants_token:
                pos = e.start + e.count
                out[e.request.id] = self.stop_at.get((e.request.id, pos), (hash((str(e.request.id), pos)) % 1000) + 10)
        self.cache.audit()
        return out


def make(n_pages=64, page=4, max_requests=4, max_req_tokens=128, budget=32, chunk=None, stop_at=None):
    cache = CacheManager([GroupSpec("full")], n_pages, page, max_requests, max_req_tokens)
    ex = FakeExecutor(cache, stop_at)
    return Scheduler(cache, ex, SchedulerParams(max_step_tokens=budget, prefill_chunk=chunk)), ex, cache


def expected_tokens(rid, n_prompt, n_new):
    return [(hash((str(rid), n_prompt + i)) % 1000) + 10 for i in range(n_new)]


def test_prompt_is_cut_under_the_budget_and_decodes_come_first():
    s, ex, cache = make(budget=10)
    s.add(Request("a", list(range(23)), max_new_tokens=3))
    s.step(); s.step()
    assert ex.plans[0] == [("a", 0, 10, False)] and ex.plans[1] == [("a", 10, 10, False)]
    s.add(Request("b", list(range(15)), max_new_tokens=2))
    s.step()                                   # a's last 3 prompt tokens, then b's first 7
    assert ex.plans[2] == [("a", 20, 3, True), ("b", 0, 7, False)]
    s.step()                                   # a decodes (1 token) before b's portion
    assert ex.plans[3] == [("a", 23, 1, True), ("b", 7, 8, True)]
    s.run_to_completion()
    assert s.finished["a"].generated == expected_tokens("a", 23, 3) and s.finished["a"].finish_reason == "length"
    assert s.finished["b"].generated == expected_tokens("b", 15, 2)
    assert cache.free_pages() == [64] and not cache.live_requests()


def test_prefill_chunk_cap_and_several_prompts_in_one_step():
    s, ex, _ = make(budget=40, chunk=24)
    for rid, n in (("a", 30), ("b", 9), ("c", 33)):
        s.add(Request(rid, list(range(n)), max_new_tokens=1))
    s.step()
    assert ex.plans[0] == [("a", 0, 24, False), ("b", 0, 9, True), ("c", 0, 7, False)]


def test_stop_ids_and_ignore_eos():
    s, ex, cache = make(stop_at={("a", 6): 2, ("b", 6): 2})
    s.add(Request("a", [1, 2, 3, 4], max_new_tokens=10, stop_ids=(2,)))
    s.add(Request("b", [1, 2, 3, 4], max_new_tokens=4, stop_ids=(2,), ignore_eos=True))
    s.run_to_completion()
    a, b = s.finished["a"], s.finished["b"]
    assert a.finish_reason == "stop" and len(a.generated) == 2 and 2 not in a.generated
    assert b.finish_reason == "length" and len(b.generated) == 4 and b.generated[2] == 2
    assert cache.free_pages() == [64]


def test_refusals_at_admission():
    s, _, _ = make(n_pages=4, page=4, max_req_tokens=64)
    with pytest.raises(ValueError, match="empty"):
        s.add(Request("e", []))
    with pytest.raises(ValueError, match="never fit"):
        s.add(Request("big", list(range(20))))             # 21 tokens need 6 pages, the pool has 4
    with pytest.raises(ValueError, match="longest request"):
        s.add(Request("long", list(range(64))))
    with pytest.raises(ValueError, match="seed 0"):
        s.add(Request("z", [1], sampling=SamplingParams(temperature=1.0, seed=0)))


def test_portion_shrinks_to_the_pages_that_are_free():
    s, ex, cache = make(n_pages=6, page=4, budget=64, max_req_tokens=24)
    s.add(Request("a", list(range(14)), max_new_tokens=50))       # 4 pages
    s.step()
    s.add(Request("b", list(range(15)), max_new_tokens=1))
    s.step()
    # 2 pages were free; one stays in hand for the live request, so the newcomer gets one page
    assert ex.plans[1] == [("a", 14, 1, True), ("b", 0, 4, False)]


def test_decode_without_pages_preempts_the_newest_request_and_it_recomputes():
    s, ex, cache = make(n_pages=8, page=4, budget=64, max_req_tokens=32)
    s.add(Request("old", list(range(12)), max_new_tokens=12))
    s.add(Request("new", list(range(100, 112)), max_new_tokens=12))
    results = {"old": [], "new": []}
    preempted_seen = False
    for _ in range(200):
        if not s.has_work():
            break
        for rid, tok, done in s.step():
            if tok is not None:
                results[rid].append(tok)
        cache.audit()
    assert s.stats["preemptions"] >= 1 and s.finished["new"].preemptions >= 1 and s.finished["old"].preemptions == 0
    # recompute: after the preemption "new" was prefilled again from position 0 with prompt + generated
    again = [p for plan in ex.plans for p in plan if p[0] == "new" and p[1] == 0]
    assert len(again) >= 2
    # and both requests got exactly the tokens they would have got alone
    assert results["old"] == expected_tokens("old", 12, 12) == s.finished["old"].generated
    assert results["new"] == expected_tokens("new", 12, 12) == s.finished["new"].generated
    assert cache.free_pages() == [8]


def test_a_lone_request_that_outgrows_the_pool_finishes_with_length():
    s, _, cache = make(n_pages=3, page=4, budget=64, max_req_tokens=64)
    s.add(Request("a", list(range(6)), max_new_tokens=100))
    s.run_to_completion()
    r = s.finished["a"]
    assert r.finish_reason == "length" and len(r.tokens) == 13 and cache.free_pages() == [3]


def test_a_request_that_planning_ends_is_reported_by_step():
    """A lone request that can get no further page is ended by the plan itself; step() says so (finished=True),
    so that a caller who follows step()'s returns sees every request end."""
    s, _, cache = make(n_pages=3, page=4, budget=64, max_req_tokens=64)
    s.add(Request("a", list(range(6)), max_new_tokens=100))
    seen = []
    while s.has_work():
        seen += s.step()
    assert seen[-1] == ("a", None, True) and sum(1 for _, _, done in seen if done) == 1
    assert [t for _, t, _ in seen if t is not None] == s.finished["a"].generated


def test_context_limit_finishes_a_request():
    s, _, _ = make(max_req_tokens=16, page=4)
    s.add(Request("a", list(range(10)), max_new_tokens=100))
    s.run_to_completion()
    assert s.finished["a"].finish_reason == "length" and len(s.finished["a"].tokens) == 16


def test_slots_limit_admission_and_order_is_first_come_first_served():
    s, ex, _ = make(max_requests=2, budget=64)
    for i in range(5):
        s.add(Request(i, list(range(5 + i)), max_new_tokens=2))
    s.step()
    assert [p[0] for p in ex.plans[0]] == [0, 1]
    s.run_to_completion()
    first_seen = []
    for plan in ex.plans:
        for p in plan:
            if p[0] not in first_seen:
                first_seen.append(p[0])
    assert first_seen == [0, 1, 2, 3, 4] and len(s.finished) == 5


@pytest.mark.parametrize("seed", range(4))
def test_random_load_with_a_starved_pool_gives_every_request_its_own_tokens(seed):
    rng = np.random.RandomState(seed)
    s, ex, cache = make(n_pages=int(rng.randint(10, 16)), page=4, max_requests=4, max_req_tokens=40,
                        budget=int(rng.randint(6, 30)), chunk=int(rng.randint(3, 12)))
    want = {}
    for i in range(12):
        n, k = int(rng.randint(1, 20)), int(rng.randint(1, 15))
        s.add(Request(i, [int(t) for t in rng.randint(0, 50, size=n)], max_new_tokens=k))
        want[i] = expected_tokens(i, n, k)
    steps = 0
    while s.has_work():
        s.step(); steps += 1
        cache.audit()
        assert steps < 5000
    for i, w in want.items():
        assert s.finished[i].generated == w, (i, s.finished[i].finish_reason)
    assert cache.free_pages() == [cache.pools[0].n_pages] and not cache.live_requests()


class PipelinedFakeExecutor(FakeExecutor):
    """The same with `launch` / `wait`, as an executor that leaves sampled ids on the device has them: a step may
    be launched before the tokens of the step ahead of it were read; an entry fed from that step carries the
    scheduler's IN_FLIGHT mark, and the token it stands for is looked up here when the step 'runs' (at wait)."""

    def __init__(self, cache, stop_at=None):
        super().__init__(cache, stop_at)
        self.launched_ahead = self.ahead_with_prompt = self.ahead_with_admission = 0

    def launch(self, plan, feed_rows=None):
        from xyntetik_runner_b200.engine.scheduler import IN_FLIGHT
        for e in plan.entries:
            fed = feed_rows is not None and e.request.id in feed_rows and e.tokens[-1] == IN_FLIGHT
            assert (IN_FLIGHT in e.tokens) == fed, "a token that is still in flight must come through the feed"
            assert not fed or e.count == 1
        self.launched_ahead += feed_rows is not None
        if feed_rows is not None:
            self.ahead_with_prompt += any(e.count > 1 or not e.wants_token for e in plan.entries)
            self.ahead_with_admission += bool(plan.admitted)
        return self.run(plan)          # commits at launch, as Engine.step does

    def wait(self, handle):
        return handle


class FailingExecutor(PipelinedFakeExecutor):
    """Refuses the launches whose numbers are in `fail_at`, the way the engine's executor does when a kernel
    refuses or the runtime fails before the step is whole: the plan's reservations are given back, then it raises."""

    def __init__(self, cache, stop_at=None, fail_at=()):
        super().__init__(cache, stop_at)
        self.fail_at, self.n_launches, self.failed = set(fail_at), 0, 0

    def launch(self, plan, feed_rows=None):
        self.n_launches += 1
        if self.n_launches in self.fail_at:
            for e in plan.entries:
                self.cache.cancel(e.request.id)
            self.failed += 1
            raise RuntimeError("injected: the step failed before it was whole")
        return super().launch(plan, feed_rows)


@pytest.mark.parametrize("ahead", [False, True])
@pytest.mark.parametrize("seed", range(4))
def test_a_step_that_fails_to_launch_changes_no_token(seed, ahead):
    """Launches fail now and then (also launches ahead of their turn, also in steps that admitted or preempted):
    the caller sees the exception, calls step() again, and every request ends with the tokens and the reason of a
    run without failures; no page is lost."""
    outcomes = []
    for fail_at in ((), (2, 3, 7, 11, 12, 20, 33, 34, 35, 50)):
        rng = np.random.RandomState(300 + seed)
        n_pages, page = int(rng.randint(14, 40)), 4
        cache = CacheManager([GroupSpec("full")], n_pages, page, 4, 60)
        sizes = [(int(rng.randint(1, 20)), int(rng.randint(1, 25))) for _ in range(10)]
        stops = {(i, sizes[i][0] + int(rng.randint(1, sizes[i][1] + 1))): 7 for i in range(0, 10, 3)}
        ex = FailingExecutor(cache, stops, fail_at)
        s = Scheduler(cache, ex, SchedulerParams(max_step_tokens=int(rng.randint(8, 30)), prefill_chunk=int(rng.randint(3, 12)),
                                                 look_ahead=ahead))
        for i, (n, k) in enumerate(sizes):
            s.add(Request(i, [int(t) for t in rng.randint(10, 50, size=n)], max_new_tokens=k, stop_ids=(7,)))
        steps = raised = 0
        while s.has_work():
            try:
                s.step()
            except RuntimeError:
                raised += 1
            steps += 1
            cache.audit()
            for r in s.live:                      # nothing reserved is left over between steps, failed or not
                assert cache.reserved(r.id) == 0 or s._ahead is not None
            assert steps < 5000
        assert cache.free_pages() == [n_pages] and not cache.live_requests()
        if fail_at:
            assert ex.failed >= 5 and raised + s.stats.get("ahead_launches_failed", 0) == ex.failed
            assert ahead == (s.stats.get("ahead_launches_failed", 0) > 0) or not ahead
        outcomes.append({i: (r.generated, r.finish_reason) for i, r in s.finished.items()})
    assert outcomes[0] == outcomes[1]


@pytest.mark.parametrize("seed", range(6))
def test_steps_launched_ahead_change_nothing(seed):
    """Random loads (starved pools, stop tokens, short and long requests) with and without looking ahead: the
    same tokens, the same reasons, every page back."""
    outcomes = []
    for ahead in (False, True):
        rng = np.random.RandomState(100 + seed)
        n_pages, page = int(rng.randint(14, 40)), 4
        cache = CacheManager([GroupSpec("full")], n_pages, page, 4, 60)
        sizes = [(int(rng.randint(1, 20)), int(rng.randint(1, 25))) for _ in range(10)]
        # every third request meets the stop token (7) somewhere among the tokens it would generate
        stops = {(i, sizes[i][0] + int(rng.randint(1, sizes[i][1] + 1))): 7 for i in range(0, 10, 3)}
        ex = PipelinedFakeExecutor(cache, stops)
        s = Scheduler(cache, ex, SchedulerParams(max_step_tokens=int(rng.randint(8, 30)), prefill_chunk=int(rng.randint(3, 12)),
                                                 look_ahead=ahead))
        for i, (n, k) in enumerate(sizes):
            s.add(Request(i, [int(t) for t in rng.randint(10, 50, size=n)], max_new_tokens=k, stop_ids=(7,)))
        steps = 0
        while s.has_work():
            s.step(); steps += 1
            cache.audit()
            assert steps < 5000
        assert cache.free_pages() == [n_pages] and not cache.live_requests()
        assert (ex.launched_ahead > 0) == ahead
        if ahead:
            # not only decode steps: steps with prompt portions, and steps that admit, are launched ahead too
            assert ex.ahead_with_prompt > 0 and ex.ahead_with_admission > 0 and ex.launched_ahead >= 0.5 * steps
        outcomes.append({i: (r.generated, r.finish_reason) for i, r in s.finished.items()})
    assert outcomes[0] == outcomes[1]
    assert any(reason == "stop" for _, reason in outcomes[0].values())


@pytest.mark.parametrize("ahead", [False, True])
def test_abort_frees_at_once_and_leaves_the_others_alone(ahead):
    cache = CacheManager([GroupSpec("full")], 64, 4, 4, 128)
    ex = PipelinedFakeExecutor(cache)
    s = Scheduler(cache, ex, SchedulerParams(max_step_tokens=32, look_ahead=ahead))
    for rid, n in (("a", 9), ("b", 5), ("c", 7), ("d", 3), ("e", 4)):
        s.add(Request(rid, list(range(10, 10 + n)), max_new_tokens=12))
    assert s.abort("e") and "e" not in [r.id for r in s.waiting]            # still waiting (four slots): leaves the queue
    assert s.finished["e"].finish_reason == "abort" and s.finished["e"].generated == []
    for _ in range(5):
        s.step()
    held = cache.free_pages()[0]
    n_b = len([r for r in s.live if r.id == "b"][0].generated)
    assert 0 < n_b < 12
    assert s.abort("b") and not s.abort("b") and not s.abort("nobody")
    assert cache.free_pages()[0] > held and "b" not in cache.live_requests()     # its pages and slot are back in this call
    cache.audit()
    s.run_to_completion()
    assert s.finished["b"].finish_reason == "abort" and s.finished["b"].generated == expected_tokens("b", 5, n_b)
    for rid, n in (("a", 9), ("c", 7), ("d", 3)):
        assert s.finished[rid].generated == expected_tokens(rid, n, 12) and s.finished[rid].finish_reason == "length"
    assert cache.free_pages() == [64] and not cache.live_requests()
    cache.audit()


def test_sampler_state_is_per_request_and_follows_the_reference_generator():
    from plain_llama import uniform_from_state, xorshift64
    s = RequestSampler(SamplingParams(temperature=0.8, seed=12345))
    st = 12345
    for _ in range(5):
        st = xorshift64(st)
        assert s.draw() == uniform_from_state(st)
    for t in range(300):
        s.accept(t)
    w = RequestSampler(SamplingParams(temperature=0.8, repeat_penalty=1.1, seed=1), no_penalty=(7,))
    for t in (5, 7, 7, 9):
        w.accept(t)
    assert sorted(x for x in w.window().tolist() if x >= 0) == [5, 9] and w.needs_window()
    assert sorted(set(s.recent.tolist())) == list(range(44, 300))
