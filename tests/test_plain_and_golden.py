"""The plain implementation: against the reference's own CPU code (golden outputs), and its own parts."""
import os

import numpy as np
import pytest

from plain_llama import (PlainLlama, attention, rope_apply, rope_inv_freq, sample_chain, softmax_rows, swiglu,
                         uniform_from_state, xorshift64)

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["GA", "GB", "GC"])
def test_plain_matches_the_reference_cpu_code(name, tmp_path):
    import sys
    sys.path.insert(0, GOLDEN)
    import golden_models as gm
    g = np.load(os.path.join(GOLDEN, f"{name}.npz"))
    assert list(g["tokens"]) == gm.token_ids(name)
    folder = gm.build_folder(str(tmp_path / name), name)
    mine = PlainLlama(folder).logits(list(g["tokens"]))[g["positions"]]
    ref = g["logits"]
    rng = float(ref.max() - ref.min())
    diff = np.abs(mine - ref)
    assert diff.mean() / rng <= 2e-3, diff.mean() / rng            # tests/test_gpu_identity.c:60
    assert diff.max() / rng <= 2e-2
    assert (mine.argmax(axis=1) == ref.argmax(axis=1)).mean() >= 0.9


def test_rotation_pairs_and_identity_at_position_zero():
    v = np.random.RandomState(0).randn(3, 2, 8).astype(np.float32)
    inv = rope_inv_freq(10000.0, 8)
    out = rope_apply(v, np.array([0, 1, 5]), inv)
    assert np.array_equal(out[0], v[0])                              # angle 0
    # norms of each pair (j, j + half) are kept
    assert np.allclose(out[..., :4] ** 2 + out[..., 4:] ** 2, v[..., :4] ** 2 + v[..., 4:] ** 2, atol=1e-5)
    # a rotation by position p then scores against position q depend on p - q only
    a = rope_apply(v[:1], np.array([7]), inv)[0, 0] @ rope_apply(v[1:2], np.array([4]), inv)[0, 0]
    b = rope_apply(v[:1], np.array([13]), inv)[0, 0] @ rope_apply(v[1:2], np.array([10]), inv)[0, 0]
    assert abs(a - b) < 1e-4


def test_attention_is_causal_grouped_and_windowed():
    rs = np.random.RandomState(1)
    q, k, v = rs.randn(6, 4, 8), rs.randn(6, 2, 8), rs.randn(6, 2, 8)
    q, k, v = (x.astype(np.float32) for x in (q, k, v))
    full = attention(q, k, v, 0.35)
    assert np.allclose(full[0, 0], v[0, 0], atol=1e-6) and np.allclose(full[0, 3], v[0, 1], atol=1e-6)   # one key; heads 2,3 -> kv 1
    k2, v2 = k.copy(), v.copy()
    k2[5], v2[5] = 9.0, -9.0
    assert np.array_equal(attention(q, k2, v2, 0.35)[:5], full[:5])  # the future does not matter
    win = attention(q, k, v, 0.35, window=2)
    assert np.allclose(win[1], full[1], atol=1e-6) and not np.allclose(win[4], full[4], atol=1e-4)
    s = (k[3:5, 0] @ q[4, 0]) * 0.35
    assert np.allclose(win[4, 0], softmax_rows(s[None])[0] @ v[3:5, 0], atol=1e-6)


def test_swiglu_and_its_floor():
    g = np.array([[-81.0, -1.0, 0.0, 2.0]], dtype=np.float32)
    u = np.array([[3.0, 3.0, 3.0, 3.0]], dtype=np.float32)
    h = swiglu(g, u)[0]
    assert h[0] == 0.0 and abs(h[1] - (-1 / (1 + np.e)) * 3) < 1e-6 and h[2] == 0.0 and abs(h[3] - 2 / (1 + np.exp(-2)) * 3) < 1e-5


def test_sampling_chain():
    lg = np.array([1.0, 3.0, 3.0, -2.0, 0.5], dtype=np.float32)
    assert sample_chain(lg, 0.0, 0.0) == 1                            # argmax, first index on ties
    assert sample_chain(lg, 0.99, 1.0, top_k=1) == 1
    # descending order is (1, 2, 0, 4, 3); with temperature 1 the first two carry 0.43 each
    assert sample_chain(lg, 0.40, 1.0) == 1 and sample_chain(lg, 0.50, 1.0) == 2 and sample_chain(lg, 0.999, 1.0) == 3
    assert sample_chain(lg, 0.999, 1.0, top_k=3) == 0
    assert sample_chain(lg, 0.999, 1.0, top_p=0.8) == 2                # prefix (1, 2) reaches 0.8
    assert sample_chain(lg, 0.999, 1.0, min_p=0.1) == 0                # 0.5 and -2 fall below a tenth of the best
    # the penalty lowers a recent positive logit and is applied once per occurrence
    assert sample_chain(lg, 0.40, 1.0, repeat_penalty=4.0, recent=[1, 1]) == 2
    assert sample_chain(lg, 0.0, 0.0, repeat_penalty=4.0, recent=[1, 2]) == 1       # greedy ignores it
    x = 88172645463325252
    x = xorshift64(x)
    assert x == 8748534153485358512 and 0.0 <= uniform_from_state(x) < 1.0


def test_score_logprobs():
    from plain_llama import score_logprobs
    lg = np.log(np.array([[0.5, 0.25, 0.25], [0.1, 0.2, 0.7], [1 / 3, 1 / 3, 1 / 3]], dtype=np.float64)).astype(np.float32) + 7.0
    lp = score_logprobs(lg, [0, 1, 2])
    assert lp.shape == (2,) and np.allclose(lp, np.log([0.25, 0.7]), atol=1e-6)
