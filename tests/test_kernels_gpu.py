"""Each kernel alone against a plain float32/float64 computation of the same op, at sizes other than the
engine's test configurations."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def bf16_round(a: torch.Tensor) -> torch.Tensor:
    return a.to(torch.bfloat16).to(torch.float32)


@pytest.mark.parametrize("n,n_out,k", [(1, 128, 64), (5, 200, 136), (16, 384, 4096), (17, 130, 72), (64, 512, 1024),
                                       (100, 256, 264), (300, 640, 512), (2, 96, 8), (200, 384, 512), (520, 100, 200), (1030, 300, 72),
                                       # more tiles than CTA pairs (80, 90, 80 and 192 on 74): the pairs walk them in rounds
                                       (1100, 4000, 512), (2300, 2560, 136), (1100, 4000, 1024), (2048, 6144, 1024),
                                       (512, 9688, 1024)])          # two tiles more than a round of 74 pairs, the last row tile ragged
@pytest.mark.parametrize("epi", ["store_bf16", "store_f32", "add", "bias"])
def test_gemm_tc(n, n_out, k, epi):
    from xyntetik_runner_b200 import kernels
    g = torch.Generator(device="cpu").manual_seed(n * 1000 + n_out + k)
    x = torch.randn(n, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(n_out, k, generator=g) / math.sqrt(k)).to(torch.bfloat16)
    bias = torch.randn(n_out, generator=g) if epi == "bias" else None
    ref = x.double() @ w.double().T
    if bias is not None:
        ref = ref + bias.double()
    xd, wd = x.to(DEV), w.to(DEV)
    bd = None if bias is None else bias.to(DEV)
    for splits in (0, 1, 3):
        if epi == "add":
            base = torch.randn(n, n_out, generator=g)
            out = base.clone().to(DEV)
            kernels.gemm_tc(xd, wd, out, bd, kernels.EPI_ADD, force_splits=splits)
            got, want, tol = out.cpu().double(), ref + base.double(), 2e-5
        elif epi == "store_bf16":
            out = torch.empty(n, n_out, dtype=torch.bfloat16, device=DEV)
            kernels.gemm_tc(xd, wd, out, bd, kernels.EPI_STORE, force_splits=splits)
            got, want, tol = out.cpu().double(), ref, 2 ** -8
        else:
            out = torch.empty(n, n_out, dtype=torch.float32, device=DEV)
            kernels.gemm_tc(xd, wd, out, bd, kernels.EPI_STORE, force_splits=splits)
            got, want, tol = out.cpu().double(), ref, 2e-5
        kernels.tc_check_status(torch.device(DEV))
        scale = float(want.abs().max())
        err = float((got - want).abs().max())
        assert err <= tol * scale, f"splits={splits}: max err {err:.3e} vs {tol * scale:.3e}"


def _activation(name, g):
    if name == "silu":
        return torch.where(g < -80, torch.zeros_like(g), g / (1 + torch.exp(-g)))
    if name == "gelu_tanh":
        return 0.5 * g * (1 + torch.tanh(0.7978845608 * (g + 0.044715 * g ** 3)))
    return g


@pytest.mark.parametrize("act", ["silu", "gelu_tanh", "none"])
@pytest.mark.parametrize("n,F,k", [(1, 128, 64), (7, 176, 72), (3, 40, 72), (5, 64, 64), (8, 200, 1024), (16, 1000, 520), (33, 300, 256), (256, 256, 128), (70, 1024, 512), (300, 200, 264), (600, 384, 128), (2500, 2000, 192), (2048, 4800, 1024), (512, 4840, 1024)])
def test_gemm_tc_gated(n, F, k, act):
    """out = act(x . W_gate) * (x . W_up) in the product's epilogue, on the packed layout that interleaves gate and
    up rows (64 features per 128-row tile), uncut and cut along K, for every activation."""
    from xyntetik_runner_b200 import kernels
    if act != "silu" and (n, F, k) not in ((7, 176, 72), (33, 300, 256), (300, 200, 264), (16, 1000, 520)):
        pytest.skip("the other activations run on a few of the sizes")
    g = torch.Generator(device="cpu").manual_seed(n + F + k)
    x = torch.randn(n, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * F, k, generator=g) * (3.0 / math.sqrt(k))).to(torch.bfloat16)
    gate = x.double() @ w[:F].double().T
    up = x.double() @ w[F:].double().T
    ref = _activation(act, gate) * up
    packed = kernels.pack_weight(w.to(DEV), halves=2)
    assert packed.shape[0] == -(-F // 64) and packed.shape[2:] == (128, 64)
    torch.cuda.synchronize()
    # (at most 16 tokens: the decode kernel, which is cut into more slices along K)
    for splits in (0, 1, 2) if n > 16 else (0, 1, 2, 3, 5, 8):
        for dt, tol in ((torch.bfloat16, 2 ** -8), (torch.float32, 3e-5 if act == "none" else 2e-3)):     # (SiLU and GELU use the hardware's approximate exp and tanh)
            out = torch.full((n, F), float("nan"), dtype=dt, device=DEV)
            kernels.gemm_tc(x.to(DEV), packed, out, None, kernels.EPI_GATED, force_splits=splits, packed_rows=F, act=kernels.ACTIVATIONS[act])
            kernels.tc_check_status(torch.device(DEV))
            err = float((out.cpu().double() - ref).abs().max())
            assert err <= tol * float(ref.abs().max()) + 1e-6, (splits, dt, err)
    with pytest.raises(kernels.KernelError):            # the gated product takes packed weights only
        kernels.gemm_tc(x.to(DEV), w.to(DEV), torch.empty(n, F, dtype=torch.bfloat16, device=DEV), None, kernels.EPI_GATED)


@pytest.mark.parametrize("act", ["silu", "gelu_tanh"])
@pytest.mark.parametrize("n,n_out,k", [(5, 200, 136), (40, 384, 1024), (300, 130, 264)])
def test_gemm_tc_store_with_activation(n, n_out, k, act):
    """out = act(x . W + bias): the epilogue of an ungated feed-forward's first product, uncut and cut along K."""
    from xyntetik_runner_b200 import kernels
    g = torch.Generator().manual_seed(n + n_out)
    x = torch.randn(n, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(n_out, k, generator=g) * (2.0 / math.sqrt(k))).to(torch.bfloat16)
    bias = torch.randn(n_out, generator=g)
    ref = _activation(act, x.double() @ w.double().T + bias.double())
    for splits in (0, 1, 3):
        out = torch.empty(n, n_out, dtype=torch.bfloat16, device=DEV)
        kernels.gemm_tc(x.to(DEV), w.to(DEV), out, bias.to(DEV), kernels.EPI_STORE, force_splits=splits, act=kernels.ACTIVATIONS[act])
        err = float((out.cpu().double() - ref).abs().max())
        assert err <= 2 ** -8 * float(ref.abs().max()) + 1e-6, (splits, err)
    kernels.tc_check_status(torch.device(DEV))


def test_gemm_tc_strided_rows_and_far_columns():
    """X rows taken out of a wider buffer (row stride > K) and a single large entry far along K."""
    from xyntetik_runner_b200 import kernels
    n, k, n_out = 9, 200, 140
    big = torch.zeros(n, 512, dtype=torch.bfloat16)
    big[:, :k] = torch.randn(n, k).to(torch.bfloat16)
    big[:, k:] = 77.0                                 # must never be read
    w = torch.zeros(n_out, k, dtype=torch.bfloat16)
    w[139, 199] = 2.0
    w[0, 0] = 1.0
    xd = big.to(DEV)[:, :k]
    out = torch.empty(n, n_out, dtype=torch.float32, device=DEV)
    kernels.gemm_tc(xd, w.to(DEV), out)
    ref = big[:, :k].double() @ w.double().T
    assert torch.equal(out.cpu().double(), ref)


@pytest.mark.parametrize("xdt,wdt,odt", [(torch.float32, torch.float32, torch.float32), (torch.float32, torch.bfloat16, torch.float32),
                                          (torch.bfloat16, torch.float32, torch.bfloat16), (torch.bfloat16, torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("n,n_out,k", [(1, 1, 1), (3, 70, 19), (65, 129, 100), (130, 64, 257)])
def test_gemm_simt(xdt, wdt, odt, n, n_out, k):
    from xyntetik_runner_b200 import kernels
    g = torch.Generator(device="cpu").manual_seed(7)
    x = torch.randn(n, k, generator=g).to(xdt)
    w = torch.randn(n_out, k, generator=g).to(wdt)
    bias = torch.randn(n_out, generator=g)
    ref = x.double() @ w.double().T + bias.double()
    out = torch.empty(n, n_out, dtype=odt, device=DEV)
    kernels.gemm_simt(x.to(DEV), w.to(DEV), out, bias.to(DEV))
    tol = 2 ** -8 if odt == torch.bfloat16 else 1e-5
    assert float((out.cpu().double() - ref).abs().max()) <= tol * float(ref.abs().max())
    if odt == torch.float32:
        acc = torch.ones(n, n_out, dtype=torch.float32, device=DEV)
        kernels.gemm_simt(x.to(DEV), w.to(DEV), acc, None, accumulate=True)
        ref2 = x.double() @ w.double().T + 1.0
        assert float((acc.cpu().double() - ref2).abs().max()) <= 1e-5 * float(ref2.abs().max())


def test_gemm_simt_is_independent_of_the_batch():
    """A token's row must be bit-identical whether it is multiplied alone or among others."""
    from xyntetik_runner_b200 import kernels
    x = torch.randn(70, 300).to(DEV)
    w = torch.randn(200, 300).to(DEV)
    full = torch.empty(70, 200, device=DEV)
    kernels.gemm_simt(x, w, full)
    for t in (0, 33, 69):
        one = torch.empty(1, 200, device=DEV)
        kernels.gemm_simt(x[t:t + 1].contiguous(), w, one)
        assert torch.equal(one[0], full[t])


@pytest.mark.parametrize("n,d", [(1, 16), (5, 100), (3, 4096), (2, 5000), (7, 5128), (3, 4090), (300, 1028), (2, 40000)])
def test_rmsnorm_and_row_gather(n, d):
    from xyntetik_runner_b200 import kernels
    x = torch.randn(n + 3, d) * 3
    w = torch.randn(d)
    eps = 3e-5
    ref = (x.double() / torch.sqrt((x.double() ** 2).mean(-1, keepdim=True) + eps)) * w.double()
    for odt, tol in ((torch.float32, 2e-6), (torch.bfloat16, 2 ** -8)):
        out = torch.empty(n + 3, d, dtype=odt, device=DEV)
        kernels.rmsnorm(x.to(DEV), w.to(DEV), out, eps)
        assert float((out.cpu().double() - ref).abs().max()) <= tol * float(ref.abs().max())
    rows = torch.tensor([n + 2, 0, 1][:min(3, n + 3)], dtype=torch.int32)
    out = torch.empty(len(rows), d, dtype=torch.float32, device=DEV)
    kernels.rmsnorm(x.to(DEV), w.to(DEV), out, eps, rows.to(DEV))
    assert float((out.cpu().double() - ref[rows.long()]).abs().max()) <= 2e-6 * float(ref.abs().max())


def test_embed_clamps_bad_ids():
    from xyntetik_runner_b200 import kernels
    table = torch.randn(50, 24).to(torch.bfloat16)
    ids = torch.tensor([3, 49, -1, 50, 0, 1000000], dtype=torch.int32)
    x = torch.empty(6, 24, device=DEV)
    kernels.embed(table.to(DEV), ids.to(DEV), x)
    want = table.float()[[3, 49, 0, 0, 0, 0]]
    assert torch.equal(x.cpu(), want)


def test_silu_mul():
    from xyntetik_runner_b200 import kernels
    n, F = 5, 176
    gu = torch.randn(n, 2 * F) * 4
    gu[0, 0], gu[0, 1], gu[0, 2] = -81.0, -79.0, 60.0
    g, u = gu[:, :F].double(), gu[:, F:].double()
    ref = torch.where(g < -80, torch.zeros_like(g), g / (1 + torch.exp(-g)) * u)
    h = torch.empty(n, F, device=DEV)
    kernels.silu_mul(gu.to(DEV), h)
    assert float((h.cpu().double() - ref).abs().max()) <= 1e-6 * float(ref.abs().max())
    assert float(h[0, 0]) == 0.0 and float(h[0, 1]) != 0.0
    # the other activations, gated and not, float32 and bfloat16, in place too
    for act in ("gelu_tanh", "none", "silu"):
        want = _activation(act, g) * u
        kernels.act_mul(gu.to(DEV), h, kernels.ACTIVATIONS[act], gated=True)
        assert float((h.cpu().double() - want).abs().max()) <= 2e-6 * float(want.abs().max()), act
        y = gu.to(DEV).to(torch.bfloat16)
        want = _activation(act, y.cpu().double())
        kernels.act_mul(y, y, kernels.ACTIVATIONS[act], gated=False)
        assert float((y.cpu().double() - want).abs().max()) <= 2 ** -8 * float(want.abs().max()), act


# ---------------------------------------------------------------------------------------------
# attention over a paged cache, against a float64 computation
# ---------------------------------------------------------------------------------------------
def _paged_case(seed, H, K, hd, page, seg_specs, dtype, window=0, spike=None, spikes=()):
    """seg_specs: [(pos0, length)].  Builds a cache with shuffled pages holding keys/values for positions
    [0, pos0 + length) of every request, and queries for the last `length` positions.  Returns everything the
    kernels need plus the float64 reference output."""
    rng = np.random.RandomState(seed)
    n_seg = len(seg_specs)
    max_len = max(p + l for p, l in seg_specs)
    max_pages = -(-max_len // page)
    n_pages = sum(-(-(p + l) // page) for p, l in seg_specs) + 3
    perm = rng.permutation(n_pages)
    cache = torch.zeros(n_pages, 1, 2, K, page, hd)
    cache.normal_()                                        # stale values everywhere: reuse must not matter
    bt = np.full((n_seg, max_pages), -1, dtype=np.int32)
    ks, vs, qs = [], [], []
    nxt = 0
    for s, (p0, L) in enumerate(seg_specs):
        T = p0 + L
        k = torch.from_numpy(rng.randn(T, K, hd).astype(np.float32))
        v = torch.from_numpy(rng.randn(T, K, hd).astype(np.float32))
        q = torch.from_numpy(rng.randn(L, H, hd).astype(np.float32))
        if spike is not None and s == spike[0]:
            # one far key stands out for the last query of this request: its value must dominate the output
            _, key_pos, strength = spike
            k[key_pos] = q[-1].reshape(K, H // K, hd)[:, 0] * strength / hd
        for seg_i, query_i, key_pos, logit in spikes:
            # key `key_pos` is made to score about `logit` against query `query_i` (first head of every kv group)
            if seg_i == s:
                k[key_pos] = q[query_i].reshape(K, H // K, hd)[:, 0] * (logit * math.sqrt(hd) / hd)
        if dtype == torch.bfloat16:
            k, v, q = bf16_round(k), bf16_round(v), bf16_round(q)
        for i in range(-(-T // page)):
            bt[s, i] = perm[nxt]; nxt += 1
        if not window:
            for i in range(-(-T // page)):                  # page by page (the same bytes as token by token below)
                t0, t1 = i * page, min(T, (i + 1) * page)
                cache[bt[s, i], 0, 0, :, :t1 - t0] = k[t0:t1].transpose(0, 1)
                cache[bt[s, i], 0, 1, :, :t1 - t0] = v[t0:t1].transpose(0, 1)
        for t in range(T if window else 0):
            if t < p0 - window + 1 - page:
                continue                                    # pages wholly behind the window may be gone
            cache[bt[s, t // page], 0, 0, :, t % page] = k[t]
            cache[bt[s, t // page], 0, 1, :, t % page] = v[t]
        if window:
            for i in range(max(0, (p0 - window + 1) // page)):
                bt[s, i] = -1
        ks.append(k); vs.append(v); qs.append(q)
    scale = 1.0 / math.sqrt(hd)
    refs = []
    G = H // K
    for (p0, L), k, v, q in zip(seg_specs, ks, vs, qs):
        out = torch.zeros(L, H, hd, dtype=torch.float64)
        for i in range(L):
            p = p0 + i
            t0 = max(0, p - window + 1) if window else 0
            for h in range(H):
                sc = (k[t0:p + 1, h // G].double() @ q[i, h].double()) * scale
                out[i, h] = torch.softmax(sc, 0) @ v[t0:p + 1, h // G].double()
        refs.append(out.reshape(L, H * hd))
    n = sum(l for _, l in seg_specs)
    qkv = torch.zeros(n, (H + 2 * K) * hd)
    qkv[:, :H * hd] = torch.cat([q.reshape(-1, H * hd) for q in qs])
    starts = np.cumsum([0] + [l for _, l in seg_specs[:-1]]).astype(np.int32)
    lens = np.array([l for _, l in seg_specs], dtype=np.int32)
    pos0 = np.array([p for p, _ in seg_specs], dtype=np.int32)
    positions = np.concatenate([np.arange(p, p + l) for p, l in seg_specs]).astype(np.int32)
    tok_seg = np.concatenate([np.full(l, s) for s, (_, l) in enumerate(seg_specs)]).astype(np.int32)
    return dict(cache=cache.to(dtype).to(DEV), bt=torch.from_numpy(bt).to(DEV), qkv=qkv.to(dtype).to(DEV),
                starts=torch.from_numpy(starts).to(DEV), lens=torch.from_numpy(lens).to(DEV), pos0=torch.from_numpy(pos0).to(DEV),
                positions=torch.from_numpy(positions).to(DEV), tok_seg=torch.from_numpy(tok_seg).to(DEV),
                ref=torch.cat(refs), n=n, n_seg=n_seg, max_pages=max_pages, max_len=max_len, lens_host=lens, scale=scale)


def _run_attention(case, kind, H, K, hd, page, window, dtype, tma=False, uneven=False):
    from xyntetik_runner_b200 import kernels
    c = case
    out = torch.zeros(c["n"], H * hd, dtype=dtype, device=DEV)
    cache = c["cache"]
    k_ptr, page_stride, v_off = cache.data_ptr(), cache.stride(0), cache.stride(2)
    qkv_dim = (H + 2 * K) * hd
    if kind == "simt":
        kernels.attention_simt(c["qkv"], qkv_dim, out, k_ptr, c["positions"], c["tok_seg"], c["bt"], page_stride, v_off,
                               H, K, hd, c["max_pages"], page, window, c["scale"])
    else:
        G = H // K
        splits = kernels.attention_mma_splits(c["max_len"], window, c["n_seg"] * K)
        pa = torch.full((c["n_seg"] * K * splits * 16 * hd,), float("nan"), device=DEV)
        pm = torch.full((c["n_seg"] * K * splits * 32,), float("nan"), device=DEV)
        lens = c["lens_host"]
        kernels.attention_mma(c["qkv"], qkv_dim, out, k_ptr, c["starts"], c["lens"], c["pos0"], c["bt"], pa, pm, page_stride,
                              v_off, H, K, hd, c["max_pages"], page, window, c["scale"], c["n_seg"], int(lens.max()),
                              c["max_len"], splits, bool((lens * G <= 16).any()), bool((lens * G > 16).any()),
                              group=(cache.data_ptr(), cache.shape[0], cache.shape[1], 0) if tma else None, uneven=uneven,
                              row_tiles=kernels.long_row_tiles(lens, G, 64) if tma else 0)      # (the row-tiled kernel's grid: exact, or an upper bound)
        kernels.tc_check_status(torch.device(DEV))
    return out.cpu().double()


ATT_CASES = [
    # H, K, hd, page, window, segments (pos0, length)
    (4, 2, 16, 16, 0, [(0, 5), (0, 70), (37, 1), (120, 9)]),
    (3, 1, 32, 8, 0, [(0, 1), (63, 2), (64, 1), (0, 129), (700, 1)]),
    (8, 2, 64, 64, 0, [(0, 200), (1500, 1), (511, 1), (512, 1), (513, 3)]),
    (32, 8, 128, 64, 0, [(0, 33), (1030, 1), (300, 70)]),
    (6, 2, 48, 4, 24, [(0, 50), (100, 1), (23, 1), (24, 1), (60, 7), (600, 2)]),
    (5, 5, 80, 16, 0, [(10, 20), (0, 3), (515, 1)]),
    (16, 1, 112, 32, 100, [(0, 10), (1100, 1), (90, 30)]),
    (12, 4, 96, 16, 0, [(5, 6), (250, 40)]),
    (8, 2, 128, 8, 0, [(0, 1), (7, 1), (8, 2), (300, 1), (1029, 1)]),
    (4, 1, 64, 16, 70, [(100, 1), (69, 1), (70, 1), (71, 1), (2100, 3)]),
    (16, 4, 128, 128, 0, [(2500, 1), (127, 1), (128, 1), (3000, 4)]),
    # enough (request, kv head) pairs that a request is cut into 2 to 8 spans, which the bulk-copy kernel combines
    # inside a cluster: requests of the same step with fewer spans than the longest (blocks without keys), with
    # one span, with several rows, and a window
    (8, 4, 128, 32, 0, [(2099, 1), (69, 1), (600, 1), (1300, 2), (63, 1), (64, 1), (2047, 1), (0, 1)]),
    (4, 4, 64, 8, 0, [(1099, 1), (500, 4), (1000, 16), (3, 2), (767, 1), (768, 1), (100, 1), (1090, 3), (0, 1), (511, 1), (512, 2), (7, 1)]),
    (16, 8, 64, 16, 1000, [(4999, 1), (900, 1), (999, 1), (1000, 2), (1001, 1), (3000, 1), (2500, 2), (40, 1)]),
    (16, 16, 64, 64, 0, [(699, 1), (5, 1), (350, 1), (351, 1), (64, 1), (698, 2), (200, 1), (0, 1)]),
    # pages of 16 and a block table of 63 entries (1,008 tokens, no multiple of the 64-key tile): the last tile of the
    # longest request would look one entry past its row of the table -- the next request's row, or past the table's
    # end for the last request -- if the copy did not stop at the row's length
    (8, 2, 64, 16, 0, [(200, 1), (999, 1)]),
    (8, 2, 128, 16, 0, [(1007, 1), (999, 1), (3, 1)]),
]


@pytest.mark.parametrize("case_id", range(len(ATT_CASES)))
@pytest.mark.parametrize("kind", ["simt_f32", "simt_bf16", "mma", "mma_tma"])
def test_attention_kernels(case_id, kind):
    H, K, hd, page, window, segs = ATT_CASES[case_id]
    dtype = torch.float32 if kind == "simt_f32" else torch.bfloat16
    case = _paged_case(case_id, H, K, hd, page, segs, dtype, window)
    if case_id >= 11:
        from xyntetik_runner_b200 import kernels
        assert 2 <= kernels.attention_mma_splits(case["max_len"], window, len(segs) * K) <= 8        # what the case is for
    got = _run_attention(case, "simt" if kind.startswith("simt") else "mma", H, K, hd, page, window, dtype, tma=kind == "mma_tma")
    ref = case["ref"]
    # inputs are exact in the kernel's own dtype, so the error is that of the arithmetic: float32 sums,
    # or (tensor-core path) probabilities rounded to bfloat16 before P.V and the bfloat16 output
    tol = 2e-5 if kind == "simt_f32" else 1.2e-2
    err = (got - ref).abs().max(dim=1).values / ref.abs().max()
    assert float(err.max()) <= tol, f"worst rows {torch.topk(err, min(5, len(err))).indices.tolist()} err {float(err.max()):.3e}"


def _even_share_segments(seed, n, longest, extras):
    rng = np.random.RandomState(seed)
    segs = [(int(p), 1) for p in rng.randint(0, longest, size=n)]
    return segs + extras


EVEN_CASES = [
    # H, K, hd, page, window, segments: more (request, kv head) pairs than three CTAs per SM, so the bulk-copy kernel cuts
    # the tiles of all pairs into even shares whatever the caller says of their lengths: requests of 1 to 80 tiles (one
    # CTA's share is about ten, so some lie inside one share, most are cut in two, the longest into many), entries of
    # two and four tokens, and prompt portions in the same step (no tiles in this kernel)
    (32, 8, 128, 64, 0, _even_share_segments(1, 49, 1400, [(5099, 1), (0, 1), (63, 1), (64, 1), (300, 2), (301, 4), (0, 40), (700, 9)])),
    # the cases below have fewer pairs (more than two an SM) and take even shares on the caller's word that the lengths are uneven
    # one query head per kv head, small pages, a window: the first tile of a request is not tile 0
    (8, 8, 64, 16, 500, _even_share_segments(2, 36, 3000, [(499, 1), (500, 1), (501, 1), (2999, 2)])),
    # fewer tiles than CTAs (most requests are prompt portions): empty shares, shares of one tile
    (16, 4, 128, 128, 0, [(int(p), 1) for p in range(0, 46)] + [(100, 1), (150, 1), (191, 1), (192, 1)] + [(10 * i, 5) for i in range(30)]),
    # head size 64, pages of 8, sixteen packed rows in some entries
    (16, 8, 64, 8, 0, _even_share_segments(4, 36, 900, [(0, 8), (100, 8), (2047, 1), (2048, 1)])),
    # about one pair per SM, lengths from 1 to 6,000 keys: even shares are taken on the caller's word that the
    # lengths are uneven; the longest request is cut into many pieces that its owner gathers
    (32, 8, 128, 32, 0, [(5999, 1), (0, 1), (3000, 2)] + [(40 * i * i, 1) for i in range(1, 12)] + [(100 + i, 1) for i in range(6)]),
]


def _random_even_case(seed):
    """Sizes drawn at random: kv heads, query heads per kv head, head size, page size, a window or none, and 24 to 60
    requests of 1 to 3,000 keys whose entries have as many tokens as 16 packed rows allow."""
    rng = np.random.RandomState(1000 + seed)
    K, G = int(rng.choice([8, 16])), int(rng.choice([1, 2, 4, 8]))
    hd, page = int(rng.choice([64, 128])), int(rng.choice([8, 16, 32, 64, 128]))
    window = int(rng.choice([0, 0, 70, 700]))
    n = int(rng.randint(24, 61)) if K == 8 else int(rng.randint(12, 31))
    segs = []
    for _ in range(n):
        L = int(rng.randint(1, 16 // G + 1)) if rng.rand() < 0.3 else 1
        top = int(rng.choice([40, 300, 3000]))
        segs.append((int(rng.randint(0, top)), L))
    return K * G, K, hd, page, window, segs


EVEN_CASES += [_random_even_case(i) for i in range(8)]


@pytest.mark.parametrize("case_id", range(len(EVEN_CASES)))
def test_decode_attention_in_even_shares(case_id):
    """Every request's last query (first head of each kv head) has ONE key, somewhere in its range, that carries most of
    its weight: a share that dropped, doubled or misplaced a tile, or an owner that missed a piece, is off by most
    of the row.  Errors are taken row by row against the row's own size."""
    from xyntetik_runner_b200 import kernels
    H, K, hd, page, window, segs = EVEN_CASES[case_id]
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    uneven = case_id > 0
    assert len(segs) * K > 3 * sms or (uneven and 8 * len(segs) * K >= 5 * sms)      # what the case is for
    rng = np.random.RandomState(100 + case_id)
    spikes = []
    for s, (p0, L) in enumerate(segs):
        p = p0 + L - 1
        first = max(0, p - window + 1) if window else 0
        spikes.append((s, L - 1, int(rng.randint(first, p + 1)), 9.0))
    case = _paged_case(200 + case_id, H, K, hd, page, segs, torch.bfloat16, window, spikes=spikes)
    even0 = kernels.attention_even_launches()
    got = _run_attention(case, "mma", H, K, hd, page, window, torch.bfloat16, tma=True, uneven=uneven)
    assert kernels.attention_even_launches() == even0 + 1
    ref = case["ref"]
    err = (got - ref).abs().max(dim=1).values / ref.abs().max(dim=1).values
    assert float(err.max()) <= 2e-2, f"worst rows {torch.topk(err, min(5, len(err))).indices.tolist()} err {float(err.max()):.3e}"
    # the flags that pieces are handed over with are lowered again, and the same launch gives the same bits
    assert int(kernels.workspace(torch.device(DEV)).flags.abs().sum()) == 0
    again = _run_attention(case, "mma", H, K, hd, page, window, torch.bfloat16, tma=True, uneven=uneven)
    assert torch.equal(got, again)
    # without the bulk copies (spans and the merge kernel) the same rows, to rounding
    other = _run_attention(case, "mma", H, K, hd, page, window, torch.bfloat16, tma=False)
    err2 = (other - ref).abs().max(dim=1).values / ref.abs().max(dim=1).values
    assert float(err2.max()) <= 2e-2


@pytest.mark.parametrize("kind", ["simt", "mma", "mma_tma"])
def test_attention_finds_a_far_key(kind):
    """One key hundreds of positions back carries almost all the weight of the last query: a kernel that
    skipped or misplaced it (a page edge, a span edge) would be far off."""
    H, K, hd, page = 8, 2, 64, 16
    for key_pos in (0, 15, 16, 511, 512, 700):
        case = _paged_case(50 + key_pos, H, K, hd, page, [(0, 3), (900, 1), (1023, 2)], torch.bfloat16, 0, spike=(1, key_pos, 60.0))
        got = _run_attention(case, kind.split("_")[0], H, K, hd, page, 0, torch.bfloat16, tma=kind.endswith("tma"))
        err = (got - case["ref"]).abs().max() / case["ref"].abs().max()
        assert float(err) <= 1.2e-2, (key_pos, float(err))


def test_decode_attention_in_spans_of_many_counts():
    """Twenty steps drawn at random (1 to 9 requests, 1 to 8 kv heads, up to 9,000 keys): the launcher cuts them into 3
    to 30 spans a request, combined inside clusters of every size up to eight or by the merge kernel.  Every request's
    query has one key that carries its weight."""
    from xyntetik_runner_b200 import kernels
    seen = set()
    for seed in range(20):
        rng = np.random.RandomState(5000 + seed)
        K, G = int(rng.choice([1, 2, 4, 8])), int(rng.choice([1, 2, 4]))
        hd, page = int(rng.choice([64, 128])), int(rng.choice([16, 64]))
        n = int(rng.randint(1, 9))
        top = int(rng.choice([600, 2500, 9000]))
        segs = [(int(rng.randint(top // 3, top)), 1) for _ in range(n)]
        if rng.rand() < 0.3:
            segs.append((int(rng.randint(0, 50)), 1))
        spikes = [(s, 0, int(rng.randint(0, p0 + 1)), 9.0) for s, (p0, L) in enumerate(segs)]
        case = _paged_case(300 + seed, K * G, K, hd, page, segs, torch.bfloat16, 0, spikes=spikes)
        seen.add(kernels.attention_mma_splits(case["max_len"], 0, len(segs) * K))
        got = _run_attention(case, "mma", K * G, K, hd, page, 0, torch.bfloat16, tma=True)
        err = (got - case["ref"]).abs().max(dim=1).values / case["ref"].abs().max(dim=1).values
        assert float(err.max()) <= 2e-2, (seed, K, G, hd, page, segs, float(err.max()))
    assert len([n for n in seen if n <= 8]) >= 4 and len([n for n in seen if n > 8]) >= 4, sorted(seen)


@pytest.mark.parametrize("key_pos", [3, 65537, 131071])
def test_decode_attention_over_a_hundred_thousand_keys(key_pos):
    """Contexts far beyond those of the other cases (Llama-3.1 allows 131,072 positions): one request with 131,072 keys
    beside requests of 40,000 and 70,002, in which ONE key -- near the start, in the middle, the very last -- carries
    nearly all the weight of the longest request's query.  Many spans and their merge in groups, page numbers in the
    thousands and rows of the cache beyond 2^19 are in play, in every decode kernel."""
    H, K, hd, page = 8, 2, 128, 64
    segs = [(131071, 1), (39999, 1), (70000, 2)]
    case = _paged_case(900 + key_pos % 7, H, K, hd, page, segs, torch.bfloat16, 0, spike=(0, key_pos, 180.0))
    ref = case["ref"]
    assert float(ref[0, :hd].abs().max()) > 0.5          # the spike row is one key's value, not a mean of thousands
    for kind in ("simt", "mma", "mma_tma", "mma_tma_even"):
        got = _run_attention(case, kind.split("_")[0], H, K, hd, page, 0, torch.bfloat16, tma="tma" in kind, uneven=kind.endswith("even"))
        err = (got - ref).abs().max(dim=1).values / ref.abs().max(dim=1).values
        assert float(err.max()) <= 2e-2, (kind, key_pos, err.tolist())


def test_prompt_attention_far_into_a_long_context():
    """A portion of 48 tokens at positions 100,000 to 100,047 on the tcgen05 kernel and on the row-tiled mma.sync kernel:
    782 tiles of 128 keys for its two row tiles, with chosen queries whose weight lies on one key near the start, in
    the middle, just before the portion and on the diagonal."""
    from xyntetik_runner_b200 import kernels
    H, K, hd, page = 8, 2, 128, 64
    p0, L = 100000, 48
    spikes = [(0, 0, 5, 16.0), (0, 17, 50000, 16.0), (0, 31, 100031, 16.0), (0, 47, 99999, 16.0)]
    c = _paged_case(77, H, K, hd, page, [(p0, L)], torch.bfloat16, 0, spikes=spikes)
    cache, ref = c["cache"], c["ref"]
    for q in (0, 17, 31, 47):
        assert float(ref[q, :hd].abs().max()) > 0.5
    out = torch.full((c["n"], H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    kernels.attention_tc(c["qkv"], out, c["starts"], c["lens"], c["pos0"], c["bt"], (cache.data_ptr(), cache.shape[0], cache.shape[1], 0),
                         H, K, hd, c["max_pages"], page, 0, c["scale"], c["n_seg"], L, row_tiles=kernels.long_row_tiles(c["lens_host"], H // K, 128))
    kernels.tc_check_status(torch.device(DEV))
    outs = {"tcgen05": out.cpu().double(), "rows": _run_attention(c, "mma", H, K, hd, page, 0, torch.bfloat16)}
    for name, got in outs.items():
        err = (got - ref).abs().max(dim=1).values / ref.abs().max(dim=1).values
        assert float(err.max()) <= 2e-2, (name, torch.topk(err, 5).indices.tolist(), float(err.max()))


@pytest.mark.parametrize("kind,hd,page", [("tc", 128, 16), ("tc", 128, 64), ("tc", 64, 32), ("rows", 128, 16), ("rows", 48, 8), ("simt", 64, 16)])
@pytest.mark.parametrize("window", [0, 100])
def test_prompt_attention_finds_keys_at_tile_page_and_window_edges(kind, hd, page, window):
    """Prompt portions (more than 16 packed rows: the tcgen05 kernel and the row-tiled mma.sync kernel).  With plain
    random keys a row's output is an average of hundreds of values and one lost key moves it by a thousandth;
    here chosen queries have ONE key that carries most of their weight -- at the first and last key of a 64- and
    128-key tile, of a page and of a copy box, on the diagonal, at position 0 -- so a kernel that drops or misplaces
    it is off by half the row.  With a window, the key at p - window + 1 must dominate and an equally strong key at
    p - window must count for nothing.  The queries sit at the first and last token of a 128-row tile of packed
    rows (four heads a token: tokens 0, 31, 32, 63 of the portion) and at its end.  Errors are taken row by row
    against that row's own size."""
    from xyntetik_runner_b200 import kernels
    H, K = 8, 2
    p0, L = 201, 300                                   # positions 201..500 are in the step, 0..200 lie in the cache
    queries = [0, 31, 32, 63, 64, 170, L - 1]
    spikes = []
    for n_q, i in enumerate(queries):
        p = p0 + i
        if window:
            spikes += [(0, i, p - window + 1, 9.0), (0, i, p - window, 9.0)]
        else:
            key = [0, 63, 64, 127, 128, p, p - 1][n_q]
            spikes.append((0, i, key, 9.0))
    case = _paged_case(7 + hd + page + window, H, K, hd, page, [(p0, L), (0, 40)], torch.bfloat16, window, spikes=spikes)
    out = torch.full((case["n"], H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    cache = case["cache"]
    if kind == "tc":
        assert kernels.attention_tc_supported(torch.bfloat16, H, K, hd, page)
        kernels.attention_tc(case["qkv"], out, case["starts"], case["lens"], case["pos0"], case["bt"],
                             (cache.data_ptr(), cache.shape[0], cache.shape[1], 0), H, K, hd, case["max_pages"], page, window,
                             case["scale"], case["n_seg"], int(case["lens_host"].max()))
        kernels.tc_check_status(torch.device(DEV))
        got = out.cpu().double()
    else:
        got = _run_attention(case, "simt" if kind == "simt" else "mma", H, K, hd, page, window, torch.bfloat16)
    ref = case["ref"]
    assert not torch.isnan(got).any()
    G = H // K
    for i in queries:
        for kvh in range(K):
            h = kvh * G                                   # the head the key was aimed at
            row_ref, row_got = ref[i, h * hd:(h + 1) * hd], got[i, h * hd:(h + 1) * hd]
            err = float((row_got - row_ref).abs().max() / row_ref.abs().max())
            assert err <= 2e-2, (kind, window, i, kvh, err)
    # and the spiked key really dominates its row in the reference (else the case would prove nothing)
    plain = _paged_case(7 + hd + page + window, H, K, hd, page, [(p0, L), (0, 40)], torch.bfloat16, window)["ref"]
    assert float((plain[queries[0], :hd] - ref[queries[0], :hd]).abs().max()) > 0.3
    # every row, against the size of the whole output
    assert float((got - ref).abs().max() / ref.abs().max()) <= 1.5e-2


@pytest.mark.parametrize("n,d", [(6, 200), (6, 1000), (3, 4096), (13, 5128), (70, 1000), (40, 4096), (64, 2048), (20, 5120), (70, 8192), (17, 1028)])
def test_fused_finishes_match_the_separate_kernels(n, d):
    """Deferred split-K products finished by the fused kernels give what product + separate kernels give
    (one block per token for narrow rows or many tokens, a cluster of blocks per token otherwise)."""
    from xyntetik_runner_b200 import kernels
    g = torch.Generator().manual_seed(3)
    k = 1024
    x_in = torch.randn(n, k, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(d, k, generator=g) / 32).to(torch.bfloat16).to(DEV)
    bias = torch.randn(d, generator=g).to(DEV)
    nw = torch.randn(d, generator=g).to(DEV)
    resid = torch.randn(n, d, generator=g).to(DEV)
    # separate: product adds into the residual, then RMSNorm
    a = resid.clone()
    kernels.gemm_tc(x_in, w, a, bias, kernels.EPI_ADD, force_splits=4)
    h_a = torch.empty(n, d, dtype=torch.bfloat16, device=DEV)
    kernels.rmsnorm(a, nw, h_a, 1e-5)
    # fused
    b = resid.clone()
    sums = kernels.gemm_tc_deferred(x_in, w, b, bias, kernels.EPI_ADD, force_splits=4)
    assert sums.splits == 4 and torch.equal(b, resid)            # nothing written yet
    h_b = torch.empty(n, d, dtype=torch.bfloat16, device=DEV)
    kernels.finish_add_rmsnorm(sums.partial, sums.splits, bias, b, nw, h_b, 1e-5)
    sums.release()
    assert torch.allclose(a, b, rtol=0, atol=1e-5 * float(a.abs().max()))
    assert float((h_a.float() - h_b.float()).abs().max()) <= 2 ** -7 * float(h_a.float().abs().max())
    # plain finish
    c = resid.clone()
    sums = kernels.gemm_tc_deferred(x_in, w, c, bias, kernels.EPI_ADD, force_splits=3)
    # a second deferred product while the first is outstanding gets a slab of its own
    other = torch.zeros(n, d, device=DEV)
    sums2 = kernels.gemm_tc_deferred(x_in, w, other, None, kernels.EPI_STORE, force_splits=2)
    assert sums2.partial.data_ptr() >= sums.partial.data_ptr() + 4 * sums.partial.numel()
    kernels.finish_plain(sums.partial, sums.splits, bias, c, True)
    kernels.finish_plain(sums2.partial, sums2.splits, None, other, False)
    sums.release(), sums2.release()
    assert torch.allclose(a, c, rtol=0, atol=1e-5 * float(a.abs().max()))
    assert torch.allclose(other + bias + resid, a, rtol=0, atol=2e-5 * float(a.abs().max()))
    assert kernels.workspace(torch.device(DEV)).live == 0 and kernels.workspace(torch.device(DEV)).top == 0


@pytest.mark.parametrize("adjacent,mscale", [(False, 1.0), (True, 1.0), (True, 0.83)])
@pytest.mark.parametrize("H,K,hd,rot", [(6, 2, 48, 48), (6, 2, 32, 32), (3, 1, 64, 32), (2, 2, 128, 128), (5, 1, 16, 16), (2, 1, 24, 20)])
@pytest.mark.parametrize("n", [5, 40])
def test_finish_rope_store_matches_rope_store(H, K, hd, rot, adjacent, mscale, n):
    """Five tokens: one block per (token, head).  Forty: the kernel with 16-byte loads where the sizes allow it (pairs
    (j, j + half), widths that are multiples of four), the same block-per-head kernel elsewhere."""
    from xyntetik_runner_b200 import kernels
    g = torch.Generator().manual_seed(4)
    page, kdim = 8, 512
    qkv_dim = (H + 2 * K) * hd
    x_in = torch.randn(n, kdim, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(qkv_dim, kdim, generator=g) / 20).to(torch.bfloat16).to(DEV)
    bias = torch.randn(qkv_dim, generator=g).to(DEV)
    if n == 5:
        positions = torch.tensor([3, 4, 5, 17, 9], dtype=torch.int32, device=DEV)
        tok_seg = torch.tensor([0, 0, 0, 1, 2], dtype=torch.int32, device=DEV)
        bt = torch.tensor([[2, 5, -1], [0, 1, 4], [6, 3, -1]], dtype=torch.int32, device=DEV)
        max_pages, n_pages = 3, 7
    else:
        runs = [(3, 17), (17, 1), (0, 9), (30, 13)]                # (first position, tokens) of four requests
        assert sum(l for _, l in runs) == n
        positions = torch.tensor([p for p0, l in runs for p in range(p0, p0 + l)], dtype=torch.int32, device=DEV)
        tok_seg = torch.tensor([s for s, (_, l) in enumerate(runs) for _ in range(l)], dtype=torch.int32, device=DEV)
        max_pages, n_pages = 6, 4 * 6 + 2
        bt = torch.randperm(n_pages, generator=g)[:4 * max_pages].reshape(4, max_pages).to(torch.int32).to(DEV)
    inv_freq = torch.rand(rot // 2, generator=g).to(DEV)
    outs = []
    for fused in (False, True):
        cache = torch.zeros(n_pages, 1, 2, K, page, hd, dtype=torch.bfloat16, device=DEV)
        qkv = torch.zeros(n, qkv_dim, dtype=torch.bfloat16, device=DEV)
        if fused:
            sums = kernels.gemm_tc_deferred(x_in, w, qkv, bias, kernels.EPI_STORE, force_splits=2)
            kernels.finish_rope_store(sums.partial, sums.splits, bias, qkv, positions, tok_seg, bt, inv_freq,
                                      cache.data_ptr(), cache.stride(0), cache.stride(2), H, K, hd, rot, max_pages, page, adjacent, mscale)
            sums.release()
        else:
            kernels.gemm_tc(x_in, w, qkv, bias, kernels.EPI_STORE, force_splits=1)
            kernels.rope_store(qkv, positions, tok_seg, bt, inv_freq, cache.data_ptr(), cache.stride(0), cache.stride(2),
                               H, K, hd, rot, max_pages, page, adjacent, mscale)
        outs.append((qkv[:, :H * hd].float().cpu(), cache.float().cpu()))
    (q0, c0), (q1, c1) = outs
    assert float(c0.abs().sum()) > 0
    # the two differ by the order of float32 sums before a bfloat16 rounding: at most one step of bfloat16
    assert float((q0 - q1).abs().max()) <= 2 ** -7 * float(q0.abs().max())
    assert float((c0 - c1).abs().max()) <= 2 ** -7 * float(c0.abs().max())
    assert torch.equal(c0 != 0, c1 != 0)                           # the same cache rows were written


@pytest.mark.parametrize("n,n_out,k", [(1, 128, 64), (8, 200, 136), (40, 384, 1024), (300, 130, 264)])
def test_gemm_tc_packed_layout(n, n_out, k):
    """The tile-packed weight layout gives bit-identical results to the plain one."""
    from xyntetik_runner_b200 import kernels
    g = torch.Generator().manual_seed(n + n_out)
    x = torch.randn(n, k, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(n_out, k, generator=g) / math.sqrt(k)).to(torch.bfloat16).to(DEV)
    packed = kernels.pack_weight(w)
    torch.cuda.synchronize()        # the product may read W before the kernel ahead of it has ended: W must be at rest
    for splits in (1, 2):
        a = torch.empty(n, n_out, dtype=torch.float32, device=DEV)
        b = torch.empty(n, n_out, dtype=torch.float32, device=DEV)
        kernels.gemm_tc(x, w, a, None, kernels.EPI_STORE, force_splits=splits)
        kernels.gemm_tc(x, packed, b, None, kernels.EPI_STORE, force_splits=splits, packed_rows=n_out)
        assert torch.equal(a, b)
    # the gated layout against the product of the plain matrix followed by the activation kernel (both round the
    # same float32 sums once, so they agree to a step of bfloat16)
    F = n_out
    w2 = (torch.randn(2 * F, k, generator=g) / math.sqrt(k)).to(torch.bfloat16).to(DEV)
    gu = torch.empty(n, 2 * F, dtype=torch.float32, device=DEV)
    a = torch.empty(n, F, dtype=torch.float32, device=DEV)
    b = torch.empty(n, F, dtype=torch.float32, device=DEV)
    kernels.gemm_tc(x, w2, gu, None, kernels.EPI_STORE, force_splits=1)
    kernels.act_mul(gu, a, kernels.ACT_SILU, gated=True)
    p2 = kernels.pack_weight(w2, halves=2)
    torch.cuda.synchronize()
    kernels.gemm_tc(x, p2, b, None, kernels.EPI_GATED, packed_rows=F, force_splits=1)
    assert float((a - b).abs().max()) <= 2e-3 * float(a.abs().max())
    kernels.tc_check_status(torch.device(DEV))


TC_ATT_CASES = [
    # H, K, page, window, segments (pos0, length)
    (32, 8, 64, 0, [(0, 200), (0, 33), (300, 70)]),
    (8, 2, 16, 0, [(0, 129), (500, 40), (127, 5)]),
    (4, 4, 8, 0, [(0, 300)]),
    (16, 1, 128, 0, [(1000, 24), (0, 9)]),
    (8, 4, 32, 100, [(0, 260), (400, 64)]),
]


@pytest.mark.parametrize("hd", [128, 64])
@pytest.mark.parametrize("case_id", range(len(TC_ATT_CASES)))
def test_attention_tc(case_id, hd):
    """Prompt attention on tcgen05 against the float64 computation (head sizes 128 and 64)."""
    from xyntetik_runner_b200 import kernels
    H, K, page, window, segs = TC_ATT_CASES[case_id]
    assert kernels.attention_tc_supported(torch.bfloat16, H, K, hd, page)
    c = _paged_case(100 + case_id + hd, H, K, hd, page, segs, torch.bfloat16, window)
    out = torch.full((c["n"], H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    cache = c["cache"]
    # (the grid is sized from the lengths, or, without them, by an upper bound whose surplus blocks return at once)
    kernels.attention_tc(c["qkv"], out, c["starts"], c["lens"], c["pos0"], c["bt"], (cache.data_ptr(), cache.shape[0], cache.shape[1], 0),
                         H, K, hd, c["max_pages"], page, window, c["scale"], c["n_seg"], int(c["lens_host"].max()),
                         row_tiles=kernels.long_row_tiles(c["lens_host"], H // K, 128) if case_id % 2 == 0 else 0)
    kernels.tc_check_status(torch.device(DEV))
    got, ref = out.cpu().double(), c["ref"]
    G = H // K
    # portions with at most 16 packed rows belong to the decode kernel: this kernel leaves them untouched
    row = 0
    for (p0, L) in segs:
        if L * G <= 16:
            assert torch.isnan(got[row:row + L]).all()
        else:
            err = (got[row:row + L] - ref[row:row + L]).abs().max(dim=1).values / ref.abs().max()
            assert float(err.max()) <= 1.2e-2, (p0, L, torch.topk(err, min(5, L)).indices.tolist(), float(err.max()))
        row += L


# ---------------------------------------------------------------------------------------------
# the sampling kernel against the plain chain
# ---------------------------------------------------------------------------------------------
def _sample_rows(logits, temp, top_k, top_p, min_p, pen, draws, recent=None, one_block=False, shortcuts=True):
    from xyntetik_runner_b200 import kernels
    rows, V = logits.shape
    f = lambda a: torch.tensor(a, dtype=torch.float32, device=DEV)
    out = torch.full((rows,), -7, dtype=torch.int32, device=DEV)
    scratch = torch.empty(rows * V, dtype=torch.float32, device=DEV)
    rec = None if recent is None else torch.tensor(recent, dtype=torch.int32, device=DEV)
    kernels.sample(torch.from_numpy(logits).to(DEV), f(temp), torch.tensor(top_k, dtype=torch.int32, device=DEV), f(top_p), f(min_p),
                   f(pen), f(draws), rec, scratch, out, one_block=one_block, shortcuts=shortcuts)
    return out.cpu().tolist()


@pytest.mark.parametrize("V,kind", [(17, "short"), (387, "short"), (1027, "short"), (5000, "short"), (16384 + 3, "short"), (128256, "short"),
                                    (131073, "short"), (17, "cluster"), (1027, "cluster"), (5000, "cluster"), (5000, "block"),
                                    (16384 + 3, "cluster"), (128256, "cluster"), (128256, "block"), (131072, "cluster"), (131073, "cluster")])
def test_sampling_kernel_matches_the_plain_chain(V, kind):
    """"short": what serving runs, one block a row that takes the reference's short cuts (top-k by selection, else the
    head of the distribution) and the long way where they do not apply (here: the rows at temperature 1.5 of the
    large vocabularies, whose head does not fit; all-equal rows; vocabularies below 4,096 without top-k).  "cluster" and
    "block": the long way for every row, in a cluster of eight blocks a row (rows of 1,025 to 131,072 values) or in one
    block.  All against the plain chain."""
    one_block, shortcuts = kind == "block", kind == "short"
    from plain_llama import sample_chain
    rng = np.random.RandomState(V)
    rows = 24
    logits = (rng.randn(rows, V) * 3).astype(np.float32)
    logits[3, :] = logits[3, 0]                         # all equal: every cut is decided by ids
    logits[4, V // 2:] = logits[4, V // 2]              # a long tie in the tail
    logits[5, 1] = logits[5].max() + 5; logits[5, 2] = logits[5, 1]      # a tie at the top
    logits[8, V - 1] = logits[8].max() + 5; logits[8, V // 3] = logits[8, V - 1]     # a greedy row: equal maxima far apart
    logits[12, :] = -np.inf; logits[12, V - 2] = -1e30                   # a greedy row: one finite value near the end
    temp = [0.0, 0.7, 1.0, 1.5] * 6
    top_k = [0, 0, 5, 40, 0, 3, 0, 1] * 3
    top_p = [1.0, 0.9, 1.0, 0.5, 0.3, 1.0, 0.95, 1.0] * 3
    min_p = [0.0, 0.0, 0.0, 0.05, 0.0, 0.0, 0.2, 0.0] * 3
    pen = [1.0, 1.3, 1.0, 1.0, 1.1, 1.0, 1.0, 2.0] * 3
    draws = [float(np.float32(x)) for x in rng.rand(rows)]
    draws[6], draws[7] = 0.0, float(np.float32(1.0 - 2 ** -24))
    recent = np.full((rows, 256), -1, dtype=np.int32)
    for r in range(rows):
        k = rng.randint(0, 60)
        recent[r, :k] = rng.randint(0, V, size=k)
        if k > 3:
            recent[r, 1] = recent[r, 0]                 # a token that occurs twice is penalised twice
    got = _sample_rows(logits, temp, top_k, top_p, min_p, pen, draws, recent, one_block=one_block, shortcuts=shortcuts)
    for r in range(rows):
        kw = dict(top_k=top_k[r], top_p=top_p[r], min_p=min_p[r], repeat_penalty=pen[r], recent=[t for t in recent[r] if t >= 0])
        want = sample_chain(logits[r], draws[r], temp[r], **kw)
        if got[r] != want:
            # float32 sums (in the short cuts: of thousands of terms, one after the other, as the reference adds them)
            # may move an edge of the cumulative distribution by a few 1e-6
            dist = sample_chain(logits[r], draws[r], temp[r], distance_of=got[r], **kw)
            assert dist <= (8e-6 if shortcuts else 2e-6), f"row {r}: kernel {got[r]}, plain {want}, draw {dist:.3e} outside the token's interval"
    # greedy rows are exact: first index among equal maxima
    for r in range(0, rows, 4):
        assert got[r] == int(np.argmax(logits[r])), f"greedy row {r}"


@pytest.mark.parametrize("V", [5, 387, 1027, 128256])
def test_logprob_kernel(V):
    """log softmax(row)[target] against float64, rows that start off a 16-byte boundary included (odd V)."""
    from xyntetik_runner_b200 import kernels
    rng = np.random.RandomState(V)
    rows = 9
    lg = (rng.randn(rows, V) * 4).astype(np.float32)
    lg[2, :] = -3.5                                      # a flat row: log(1 / V)
    lg[3, V // 2] = 60.0                                 # one value far above the rest
    target = rng.randint(0, V, size=rows).astype(np.int32)
    target[3] = V // 2
    out = torch.full((rows,), 7.0, dtype=torch.float32, device=DEV)
    kernels.logprob(torch.from_numpy(lg).to(DEV), torch.from_numpy(target).to(DEV), out)
    x = lg.astype(np.float64)
    m = x.max(axis=1, keepdims=True)
    ref = x[np.arange(rows), target] - (m[:, 0] + np.log(np.exp(x - m).sum(axis=1)))
    assert np.abs(out.cpu().numpy() - ref).max() <= 2e-6 * max(1.0, float(np.abs(ref).max()))
    assert abs(float(out[2]) + np.log(V)) <= 1e-5 and abs(float(out[3])) <= 1e-6


def test_sampling_kernel_follows_the_distribution():
    """Many draws at one row: empirical frequencies of the kept tokens match softmax(logits / temp)."""
    V, n = 50, 4000
    rng = np.random.RandomState(1)
    base = (rng.randn(V) * 2).astype(np.float32)
    logits = np.tile(base, (n, 1))
    draws = [float(np.float32(x)) for x in rng.rand(n)]
    got = np.array(_sample_rows(logits, [0.9] * n, [10] * n, [1.0] * n, [0.0] * n, [1.0] * n, draws))
    order = np.argsort(-base)[:10]
    p = np.exp((base[order] - base[order[0]]) / 0.9); p /= p.sum()
    assert set(got.tolist()) <= set(order.tolist())
    freq = np.array([(got == t).mean() for t in order])
    assert np.abs(freq - p).max() < 4 * np.sqrt(0.25 / n)


@pytest.mark.parametrize("shortcuts", [True, False])
def test_sampling_with_a_window_token_that_is_still_on_the_device(shortcuts):
    """A step queued before the host has read the step before it: the window of recent tokens that the host sends lacks
    one token, which lies in the array of sampled ids on the device.  The kernel puts it into the entry the host names,
    unless it is one of the row's exempt ids; the picks are those of the complete window."""
    from xyntetik_runner_b200 import kernels
    rng = np.random.RandomState(5)
    rows, V = 12, 5003
    logits = (rng.randn(rows, V) * 2).astype(np.float32)
    f = lambda a: torch.tensor(a, dtype=torch.float32, device=DEV)
    temp, top_k, top_p, min_p, pen = [0.9] * rows, [0, 40, 7] * 4, [0.9, 1.0] * 6, [0.0] * rows, [1.6, 0.7, 1.0] * 4
    draws = [float(np.float32(x)) for x in rng.rand(rows)]
    complete = np.full((rows, 256), -1, dtype=np.int32)
    partial, pending = complete.copy(), np.full((rows, 3), -1, dtype=np.int32)
    exempt = np.full((rows, kernels.EXEMPT_IDS), -1, dtype=np.int32)
    feed = rng.randint(0, V, size=64).astype(np.int32)
    for r in range(rows):
        n = int(rng.randint(3, 250))
        best = np.argsort(-logits[r])[:6]
        complete[r, :n] = rng.choice(np.concatenate([best, rng.randint(0, V, size=20)]), size=n)
        partial[r] = complete[r]
        if r % 4 != 3:                                     # (every fourth row: nothing is pending)
            slot, j = int(rng.randint(0, 256)), int(rng.randint(0, 64))
            feed[j] = best[r % 6]                          # the token on the device is one of the likeliest: it matters
            partial[r, slot] = int(rng.randint(0, V))      # what the host has there is the entry's old content
            complete[r, slot] = feed[j]
            pending[r] = (j, slot, 0)
            if r % 4 == 2:                                 # ... and here it is exempt: the complete window has no entry for it
                exempt[r, :3] = (int(rng.randint(0, V)), feed[j], 11)
                pending[r, 2] = 3
                complete[r, slot] = -1
    outs = []
    for window, pend in ((complete, None), (partial, pending)):
        out = torch.full((rows,), -7, dtype=torch.int32, device=DEV)
        scratch = torch.empty(rows * V, dtype=torch.float32, device=DEV)
        i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
        kernels.sample(torch.from_numpy(logits).to(DEV), f(temp), torch.tensor(top_k, dtype=torch.int32, device=DEV), f(top_p), f(min_p),
                       f(pen), f(draws), i32(window), scratch, out, shortcuts=shortcuts,
                       pending=None if pend is None else i32(pend), feed=None if pend is None else i32(feed),
                       exempt=None if pend is None else i32(exempt))
        outs.append(out.cpu().tolist())
    assert outs[0] == outs[1]
    assert len(set(outs[0])) > 3 and min(outs[0]) >= 0
