"""Each part of a layer alone (norm, position encoding + cache store, attention, feed-forward, block,
embedding and head), driven through its own interface, against the plain functions."""
import numpy as np
import pytest
import torch

import tiny
from plain_llama import PlainLlama, attention, embed, matvec_rows, rmsnorm, rope_apply, swiglu

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def setup(tmp_path_factory):
    out = {}
    for name in "BC":
        for dt in ("float32", "bfloat16"):
            folder = tiny.make_folder(str(tmp_path_factory.mktemp(f"p{name}{dt}")), name, dt)
            out[name, dt] = folder
    return out


def make_ctx(eng, portions):
    """portions: [(request, n_tokens)]; returns the step context the parts see."""
    from xyntetik_runner_b200.engine.engine import StepEntry
    entries = []
    for rid, n in portions:
        if not eng.cache.is_open(rid):
            eng._open(rid)
        eng.cache.reserve(rid, n)
        entries.append(StepEntry(rid, [0] * n, []))
    ctx = eng._describe(entries)
    return ctx, entries


def commit(eng, entries):
    for e in entries:
        eng.cache.commit(e.request)


TOL = {"float32": 2e-5, "bfloat16": 2e-2}


def close(got, ref, dtype, what):
    got, ref = got.float().cpu().numpy().astype(np.float64), np.asarray(ref, dtype=np.float64)
    err = np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-9)
    assert err <= TOL[dtype], f"{what}: {err:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "C"])
def test_parts_alone(setup, name, dtype):
    from xyntetik_runner_b200.engine.engine import Engine, EngineParams
    folder = setup[name, dtype]
    plain = PlainLlama(folder)
    w, cfg = plain.w, tiny.CONFIGS[name]
    d, T = cfg["hidden_size"], 53
    eng = Engine(folder, EngineParams(dtype=dtype, max_tokens=256, page_size=8, max_requests=2))
    act = eng.act_dtype
    g = torch.Generator().manual_seed(1)
    block = eng.plan.blocks[1]
    p = "model.layers.1."
    lay = eng.model.layers[1]
    x0 = (torch.randn(T, d, generator=g) * 2).to("cuda")
    x0_np = x0.cpu().numpy()

    # --- norm ---
    ctx, entries = make_ctx(eng, [("a", T)])
    h = torch.empty(T, d, dtype=act, device="cuda")
    block.mixer_norm.forward(ctx, x0, h)
    h_ref = rmsnorm(x0_np, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
    close(h, h_ref, dtype, "norm")
    rows = torch.tensor([5, 0, 52], dtype=torch.int32, device="cuda")
    h3 = torch.empty(3, d, dtype=act, device="cuda")
    block.mixer_norm.forward(ctx, x0, h3, rows=rows)
    close(h3, h_ref[[5, 0, 52]], dtype, "norm rows")

    # --- feed-forward: adds into the residual stream ---
    hin = h.clone()
    x = x0.clone()
    block.feed_forward.forward(ctx, hin, x)
    ctx.materialize(x)
    hin_np = hin.float().cpu().numpy()
    ff_ref = matvec_rows(swiglu(matvec_rows(hin_np, w[p + "mlp.gate_proj.weight"]), matvec_rows(hin_np, w[p + "mlp.up_proj.weight"])),
                         w[p + "mlp.down_proj.weight"])
    close(x, x0_np + ff_ref, dtype, "feed-forward")

    # --- mixer (attention with its position encoding and the cache store): whole, then as two portions ---
    def mixer_ref(hn):
        H, K, hd = plain.H, plain.K, plain.hd
        b = (lambda n: w.get(p + n)) if cfg.get("attention_bias") else (lambda n: None)
        q = matvec_rows(hn, w[p + "self_attn.q_proj.weight"], b("self_attn.q_proj.bias")).reshape(-1, H, hd)
        k = matvec_rows(hn, w[p + "self_attn.k_proj.weight"], b("self_attn.k_proj.bias")).reshape(-1, K, hd)
        v = matvec_rows(hn, w[p + "self_attn.v_proj.weight"], b("self_attn.v_proj.bias")).reshape(-1, K, hd)
        pos = np.arange(hn.shape[0])
        q, k = rope_apply(q, pos, plain.inv_freq), rope_apply(k, pos, plain.inv_freq)
        o = attention(q, k, v, plain.scale, plain._window(1)).reshape(-1, H * hd)
        return matvec_rows(o, w[p + "self_attn.o_proj.weight"], b("self_attn.o_proj.bias"))
    att_ref = mixer_ref(hin_np)
    x = torch.zeros(T, d, device="cuda")
    block.mixer.forward(ctx, hin, x, lay)
    ctx.materialize(x)
    close(x, att_ref, dtype, "attention whole")
    commit(eng, entries)
    eng.end("a")
    T1 = 30
    ctx, entries = make_ctx(eng, [("b", T1)])
    x1 = torch.zeros(T1, d, device="cuda")
    block.mixer.forward(ctx, hin[:T1].contiguous(), x1, lay)
    ctx.materialize(x1)
    commit(eng, entries)
    ctx, entries = make_ctx(eng, [("b", T - T1)])
    x2 = torch.zeros(T - T1, d, device="cuda")
    block.mixer.forward(ctx, hin[T1:].contiguous(), x2, lay)
    ctx.materialize(x2)
    commit(eng, entries)
    close(torch.cat([x1, x2]), att_ref, dtype, "attention in two portions")
    eng.end("b")

    # --- the block: norm, mixer, +x, norm, feed-forward, +x ---
    ctx, entries = make_ctx(eng, [("c", T)])
    x = x0.clone()
    block.forward(ctx, x, lay)
    ctx.materialize(x)
    close(x, plain.layer(x0_np, 1, np.arange(T)), dtype, "block")
    commit(eng, entries)

    # --- embedding and head ---
    ids = torch.tensor([3, 0, cfg["vocab_size"] - 1, cfg["vocab_size"] + 5, -2], dtype=torch.int32, device="cuda")
    e = torch.empty(5, d, device="cuda")
    eng.plan.embedding.forward(ctx, ids, e)
    close(e, embed(ids.cpu().numpy(), w["model.embed_tokens.weight"]), dtype, "embedding")
    hh = h[:4].contiguous()
    logits = torch.empty(4, cfg["vocab_size"], device="cuda")
    eng.plan.head.forward(ctx, hh, logits)
    close(logits, matvec_rows(hh.float().cpu().numpy(), w["lm_head.weight"]), dtype, "head")
    eng.end("c")


@pytest.mark.parametrize("adjacent,mscale", [(False, 1.0), (True, 1.0), (False, 1.3), (True, 0.7)])
@pytest.mark.parametrize("dtype,hd,rot", [(torch.float32, 80, 48), (torch.bfloat16, 80, 48), (torch.bfloat16, 72, 40),
                                          (torch.bfloat16, 128, 128), (torch.bfloat16, 64, 0), (torch.float32, 25, 10),
                                          (torch.bfloat16, 100, 100)])
def test_rotation_and_store_kernel_at_other_sizes(dtype, hd, rot, adjacent, mscale):
    """rope_store with a partial rotary dimension and odd page size against the plain rotation: float32, and
    bfloat16 on its 16-byte vector path (head size a multiple of 8, rotated width of 16) and off it; pairs
    (j, j + half) and adjacent pairs (2j, 2j + 1); cosines and sines scaled by mscale."""
    from plain_llama import rope_inv_freq
    from xyntetik_runner_b200 import kernels
    H, K, page, n = 5, 1, 5, 9
    rng = np.random.RandomState(0)
    qkv = rng.randn(n, (H + 2 * K) * hd).astype(np.float32)
    qkv = torch.from_numpy(qkv).to(dtype).float().numpy()            # values the dtype holds exactly
    tol = 1e-5 if dtype == torch.float32 else 2.0 ** -8 * 6
    positions = np.array([0, 1, 2, 3, 4, 5, 6, 300, 301], dtype=np.int32)
    tok_seg = np.array([0] * 7 + [1, 1], dtype=np.int32)
    bt = np.full((2, 62), -1, dtype=np.int32)
    bt[0, :2] = [3, 1]
    bt[1, 60] = 0
    inv = rope_inv_freq(1234.5, rot) if rot else np.zeros(0, dtype=np.float32)
    cache = torch.zeros(4, 1, 2, K, page, hd, device="cuda", dtype=dtype)
    t = torch.from_numpy(qkv).cuda().to(dtype)
    kernels.rope_store(t, torch.from_numpy(positions).cuda(), torch.from_numpy(tok_seg).cuda(), torch.from_numpy(bt).cuda(),
                       torch.from_numpy(inv).cuda() if rot else None, cache.data_ptr(), cache.stride(0), cache.stride(2),
                       H, K, hd, rot, 62, page, adjacent, mscale)
    q_ref = qkv[:, :H * hd].reshape(n, H, hd).copy()
    k_ref = qkv[:, H * hd:(H + K) * hd].reshape(n, K, hd).copy()
    if rot:
        q_ref[:, :, :rot] = rope_apply(q_ref[:, :, :rot], positions, inv, adjacent, mscale)
        k_ref[:, :, :rot] = rope_apply(k_ref[:, :, :rot], positions, inv, adjacent, mscale)
    got = t.float().cpu().numpy()
    assert np.abs(got[:, :H * hd].reshape(n, H, hd) - q_ref).max() < tol
    c = cache.float().cpu().numpy()
    for i in range(n):
        pg = bt[tok_seg[i], positions[i] // page]
        assert np.abs(c[pg, 0, 0, :, positions[i] % page] - k_ref[i]).max() < tol
        assert np.array_equal(c[pg, 0, 1, :, positions[i] % page], qkv[i, (H + K) * hd:].reshape(K, hd))
    assert np.count_nonzero(c) == n * 2 * K * hd                      # nothing else was written
