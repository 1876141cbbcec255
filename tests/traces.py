"""Traces for the replay tests: the same requests cut in different ways, and the comparison."""
import numpy as np


def random_tokens(seed, n, vocab):
    return [int(t) for t in np.random.RandomState(seed).randint(0, vocab, size=n)]


def whole(requests):
    """Each request alone and whole, logits at every position.  requests: {id: tokens}."""
    steps = []
    for k, (rid, toks) in enumerate(requests.items()):
        steps.append({"step": k, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps


def tail_decoded(requests, tail=32):
    """Most of each request in one step, the last `tail` tokens one by one."""
    steps, k = [], 0
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": k, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        k += 1
        for i in range(head, len(toks)):
            steps.append({"step": k, "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}],
                          "end": [rid] if i == len(toks) - 1 else []})
            k += 1
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def portions(requests, sizes=(7, 3, 2, 13, 2, 5, 1, 17, 2, 4)):
    """Portions of changing size, down to two tokens (and one), one request at a time."""
    steps, k = [], 0
    for rid, toks in requests.items():
        at, j = 0, 0
        while at < len(toks):
            m = min(sizes[j % len(sizes)], len(toks) - at)
            steps.append({"step": k, "entries": [{"id": rid, "tokens": toks[at:at + m], "want": list(range(m))}],
                          "end": [rid] if at + m == len(toks) else []})
            at += m
            j += 1
            k += 1
    return steps


def mixed(requests, seed=0, max_live=4, sizes=(1, 1, 2, 5, 1, 9, 3, 1, 16, 2), skip_prob=0.2):
    """Up to `max_live` requests live at a time, portions of some beside single tokens of others; a request
    is sometimes left out of a step; finished requests end so that their pages are used again."""
    rng = np.random.RandomState(seed)
    waiting = list(requests.items())
    live = {}            # rid -> [tokens, at]
    steps, k = [], 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live[rid] = [toks, 0]
        entries, ended = [], []
        for rid in list(live):
            toks, at = live[rid]
            if len(live) > 1 and rng.rand() < skip_prob:
                continue
            m = min(int(sizes[rng.randint(len(sizes))]), len(toks) - at)
            entries.append({"id": rid, "tokens": toks[at:at + m], "want": list(range(m))})
            live[rid][1] = at + m
            if at + m == len(toks):
                ended.append(rid)
                del live[rid]
        if entries:
            steps.append({"step": k, "entries": entries, "end": ended})
            k += 1
    return steps


def collect(steps, results, vocab):
    """Reassemble {request id: [positions, vocab]} from the step outputs (all positions wanted)."""
    out = {}
    for st in steps:
        if st["step"] not in results:
            continue
        arr = results[st["step"]].reshape(-1, vocab)
        at = 0
        for e in st["entries"]:
            w = len(e["want"])
            out.setdefault(e["id"], []).append(arr[at:at + w])
            at += w
        assert at == arr.shape[0]
    return {rid: np.concatenate(parts, axis=0) for rid, parts in out.items()}


def pool_tokens(steps, round_to=64):
    """The most tokens live requests hold at any time, each rounded up to a multiple of `round_to`."""
    held, peak = {}, 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-v // round_to) * round_to for v in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return peak


# Tolerances, fixed before the first run.
#  float32: every value is float32 with float32 accumulation against a float64-accumulated plain
#  implementation; a few dozen roundings of 6e-8 relative each on values of the logits' size.
#  bfloat16: activations and cached keys/values are rounded to 8 bits of mantissa (2^-9 relative) at
#  every product's input; the error of a logit is a sum of many such roundings.
TOL = {"float32": dict(max_rel=5e-5, mean_rel=5e-6), "bfloat16": dict(max_rel=6e-2, mean_rel=1e-2)}


def assert_close(got, ref, dtype, what=""):
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    scale = float(np.abs(ref).max())
    diff = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    tol = TOL[dtype]
    worst = np.unravel_index(int(diff.argmax()), diff.shape)
    row_err = diff.max(axis=1) / scale
    bad_rows = np.nonzero(row_err > tol["max_rel"])[0]
    assert diff.max() <= tol["max_rel"] * scale, (
        f"{what}: max |diff| {diff.max():.3e} > {tol['max_rel']:.1e} * {scale:.3f} at position {worst[0]}, "
        f"token {worst[1]}; first wrong position {bad_rows[0] if len(bad_rows) else None}, "
        f"wrong positions {bad_rows[:20].tolist()}")
    assert diff.mean() <= tol["mean_rel"] * scale, f"{what}: mean |diff| {diff.mean():.3e} > {tol['mean_rel']:.1e} * {scale:.3f}"
