"""The two native libraries build here (nvcc cross-compiles for sm_100a without a GPU) and export what the Python
side declares."""
import ctypes


def test_cuda_library_exports_every_declared_launcher():
    from xyntetik_runner_b200 import kernels
    lib = kernels.lib()                    # compiles on first use; _declare() touches every symbol it names
    for name in ("xr_gemm_tc", "xr_gemm_tc_noalloc", "xr_attention_tc", "xr_attention_mma", "xr_sample", "xr_sample_one_block",
                 "xr_logprob", "xr_rmsnorm", "xr_rope_store", "xr_embed", "xr_finish_add_rmsnorm"):
        assert isinstance(getattr(lib, name), ctypes._CFuncPtr), name
    assert lib.xr_attention_tc_supported(32, 8, 128, 64) == 1 and lib.xr_attention_tc_supported(32, 8, 64, 64) == 1
    assert lib.xr_attention_tc_supported(32, 8, 96, 64) == 0 and lib.xr_attention_tc_supported(32, 8, 128, 48) == 0


def test_host_library_exports_the_cache_manager():
    from xyntetik_runner_b200.cache.pages import host_lib
    lib = host_lib()
    for name in ("xrh_cache_create", "xrh_reserve", "xrh_commit", "xrh_cancel", "xrh_close", "xrh_audit", "xrh_describe"):
        assert isinstance(getattr(lib, name), ctypes._CFuncPtr), name
