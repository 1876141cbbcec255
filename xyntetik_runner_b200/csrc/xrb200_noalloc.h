/* An entry point of libxrb200.so that allocates no memory.  It has no counterpart in the reference.
 *
 * Who needs it.  Some programs that want this library's tensor-core matrix product cannot let it call
 * cudaMalloc, or hand it a workspace of their own: a host application that gave all device memory to its own
 * arena at start-up and forbids allocation afterwards; a real-time loop on a thread that must never block on
 * the driver's allocator (cudaMalloc and cudaFree may synchronise the whole device); a plug-in interface that
 * passes input and output buffers and nothing else.  For them the product's split-K scratch (float32
 * partial sums, one slab per K split) and its status word live in arrays that are part of the library's
 * image on the device.
 *
 *   int xr_gemm_tc_noalloc(X, W, bias, out, out_dtype, epilogue, n, n_out, K, ldx, ldo, status_out_host, stream)
 *
 * computes  out[t][r] = sum_k X[t][k] * W[r][k]  exactly as xr_gemm_tc does when it is given all the scratch it
 * may want: the same kernels and the same cut along K (one planner decides for both entry points, for every
 * number of tokens), so the same bits:
 *   X        [n, K] bfloat16, row stride ldx elements (a multiple of 8), 16-byte aligned
 *   W        [n_out, K] bfloat16, dense
 *   bias     [n_out] float32 or NULL
 *   out      [n, n_out], row stride ldo; out_dtype 0 = float32, 1 = bfloat16
 *   epilogue 0 = store, 1 = add into a float32 `out`  (the gated product needs weights in the library's packed
 *            layout and is not offered here)
 *   status_out_host  NULL, or a host int: the call then waits for the product and stores 0, or 1 if a
 *            bounded wait inside a kernel gave up (the output is then not valid)
 *   returns 0, or: -1 sizes/alignment/epilogue the entry point refuses (checked before anything is queued);
 *            -2 CUDA refused a launch; -3 tensor-map encoding failed; -4 the cut that the product would choose
 *            needs more split-K scratch than the fixed array holds (xr_gemm_tc_noalloc_max_floats() float32 values;
 *            the need is splits * n * n_out) -- the call is refused rather than run with another cut, whose sums
 *            would round differently from what xr_gemm_tc gives; products that are not cut (most products of more
 *            than a few hundred tokens) need no scratch and are never refused for it;
 *            -5 set-up failed (no current device, or the array's address could not be resolved).
 *
 * Rules that come with a scratch that nobody allocates:
 *  - The array is 16 MiB of every GPU's memory from the moment the library is loaded there until the process
 *    exits, whether or not this entry point is ever called.
 *  - The first call on a device resolves the array's device address (cudaGetSymbolAddress, with that device
 *    current) and keeps it; make that first call outside any stream capture.
 *  - All calls on a device share the array, and it keeps what the last call left.  The status word is cleared
 *    at the start of each call; the partial sums need no clearing because each call writes every value it
 *    later reads.  Two calls that may run on the GPU at the same time (different streams, no dependency)
 *    would overwrite each other's partial sums: order them, or use xr_gemm_tc with a scratch per stream.
 *  - Nothing in the call allocates or frees: no cudaMalloc, cudaFree, or library routine that does.
 */
#ifndef XRB200_NOALLOC_H
#define XRB200_NOALLOC_H
#include <cuda_runtime.h>
#ifdef __cplusplus
extern "C" {
#endif
int xr_gemm_tc_noalloc(const void* X, const void* W, const float* bias, void* out, int out_dtype, int epilogue,
                       int n, int n_out, int K, long long ldx, long long ldo, int* status_out_host,
                       cudaStream_t stream);
long long xr_gemm_tc_noalloc_max_floats(void);
#ifdef __cplusplus
}
#endif
#endif
