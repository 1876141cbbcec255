"""The library's allocation-free entry point, called through its exported C symbol.

Some callers of the tensor-core product may not allocate device memory (a host program with a fixed arena,
a loop that must not block on the driver's allocator, an interface that passes inputs and outputs only).
`xr_gemm_tc_noalloc` keeps its split-K scratch in an array inside the library.  This test calls it twice in a
row -- the second call finds the first call's partial sums in the shared array -- and compares both results
with the ordinary entry point's.  It is collected last, so a run that stops at the first failure has run
every other test before it.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_no_alloc_entry_point_matches_the_ordinary_one_twice():
    from xyntetik_runner_b200 import kernels
    lib = ctypes.CDLL(kernels.library_file())
    fn = lib.xr_gemm_tc_noalloc
    vp, i, ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    fn.argtypes = [vp, vp, vp, vp, i, i, i, i, i, ll, ll, ctypes.POINTER(ctypes.c_int), vp]
    fn.restype = ctypes.c_int
    lib.xr_gemm_tc_noalloc_max_floats.restype = ll
    assert lib.xr_gemm_tc_noalloc_max_floats() == 4 << 20

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator().manual_seed(11)
    # shapes whose products are cut along K (few output tiles, long K), so the scratch is really used -- at up to 16
    # tokens, in the 129..256-token range and beyond 256 tokens, where the CTA-pair kernel runs and cuts by its own
    # rule -- and one that is not cut at all
    cases = [(8, 512, 4096, 0, torch.bfloat16), (5, 256, 2048, 1, torch.float32), (8, 512, 4096, 0, torch.bfloat16),
             (200, 1024, 8192, 0, torch.bfloat16), (256, 2048, 4096, 1, torch.float32), (300, 512, 8192, 0, torch.float32),
             (700, 4096, 512, 0, torch.bfloat16), (200, 1024, 8192, 0, torch.bfloat16),
             (512, 9688, 1024, 1, torch.float32)]            # (two tiles more than a round of the CTA pairs)
    cut = 0
    for call, (n, n_out, k, epi, out_dt) in enumerate(cases):
        x = torch.randn(n, k, generator=g).to(torch.bfloat16).to(dev)
        w = (torch.randn(n_out, k, generator=g) / math.sqrt(k)).to(torch.bfloat16).to(dev)
        base = torch.randn(n, n_out, generator=g).to(out_dt).to(dev)
        want = base.clone()
        cut += kernels.gemm_tc(x, w, want, None, epi) > 1           # the existing entry point
        got = base.clone()
        status = ctypes.c_int(-1)
        rc = fn(x.data_ptr(), w.data_ptr(), None, got.data_ptr(), 0 if out_dt == torch.float32 else 1, epi, n, n_out, k,
                x.stride(0), got.stride(0), ctypes.byref(status), stream)
        assert rc == 0 and status.value == 0, (call, rc, status.value)
        torch.cuda.synchronize()
        ref = x.double().cpu() @ w.double().cpu().T
        if epi == 1:
            ref = ref + base.double().cpu()
        tol = 2e-5 if out_dt == torch.float32 else 2 ** -8
        assert float((got.double().cpu() - ref).abs().max()) <= tol * float(ref.abs().max()), call
        assert torch.equal(got, want), call                          # same kernels, same cut: same bits
    assert cut >= 5                                                  # most of them did use the scratch
    # A product whose cut needs more partial sums than the array holds is refused, and says so.  Which products
    # are cut is the planner's business: the ordinary entry point reports the cut it made.
    limit = lib.xr_gemm_tc_noalloc_max_floats()
    refused = 0
    for n, n_out, k in ((256, 8448, 8192), (128, 16384, 16384)):
        x = torch.zeros(n, k, dtype=torch.bfloat16, device=dev)
        w = torch.zeros(n_out, k, dtype=torch.bfloat16, device=dev)
        out = torch.zeros(n, n_out, dtype=torch.bfloat16, device=dev)
        splits = kernels.gemm_tc(x, w, out, None, 0)
        rc = fn(x.data_ptr(), w.data_ptr(), None, out.data_ptr(), 1, 0, n, n_out, k, k, n_out, None, stream)
        assert rc == (-4 if splits > 1 and splits * n * n_out > limit else 0), (n, n_out, k, splits, rc)
        refused += rc == -4
        del x, w, out
    assert refused >= 1
    # refusals of arguments come before anything is queued: no tokens, K not a multiple of 8, the gated epilogue
    x = torch.zeros(8, 64, dtype=torch.bfloat16, device=dev)
    w = torch.zeros(128, 64, dtype=torch.bfloat16, device=dev)
    out = torch.zeros(8, 128, dtype=torch.bfloat16, device=dev)
    assert fn(x.data_ptr(), w.data_ptr(), None, out.data_ptr(), 1, 0, 0, 128, 64, 64, 128, None, stream) == -1
    assert fn(x.data_ptr(), w.data_ptr(), None, out.data_ptr(), 1, 0, 8, 128, 60, 64, 128, None, stream) == -1
    assert fn(x.data_ptr(), w.data_ptr(), None, out.data_ptr(), 1, 2, 8, 64, 64, 64, 64, None, stream) == -1
