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
                                       (100, 256, 264), (300, 640, 512), (2, 96, 8)])
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


@pytest.mark.parametrize("n,F,k", [(1, 128, 64), (7, 176, 72), (33, 300, 256), (256, 256, 128), (70, 1024, 512)])
def test_gemm_tc_swiglu(n, F, k):
    from xyntetik_runner_b200 import kernels
    g = torch.Generator(device="cpu").manual_seed(n + F + k)
    x = torch.randn(n, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * F, k, generator=g) * (3.0 / math.sqrt(k))).to(torch.bfloat16)
    gate = x.double() @ w[:F].double().T
    up = x.double() @ w[F:].double().T
    ref = gate / (1 + torch.exp(-gate)) * up
    for splits in (0, 1, 2):
        out = torch.empty(n, F, dtype=torch.bfloat16, device=DEV)
        kernels.gemm_tc(x.to(DEV), w.to(DEV), out, None, kernels.EPI_SWIGLU, force_splits=splits)
        kernels.tc_check_status(torch.device(DEV))
        err = float((out.cpu().double() - ref).abs().max())
        assert err <= 2 ** -8 * float(ref.abs().max()) + 1e-6, (splits, err)


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


@pytest.mark.parametrize("n,d", [(1, 16), (5, 100), (3, 4096), (2, 5000)])
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
