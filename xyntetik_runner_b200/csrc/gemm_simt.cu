// out[t][r] = sum_k X[t][k] * W[r][k] (+ bias[r]) on CUDA cores with float32
// FMA: the matrix product of the true 32-bit path, and of any weight the
// tensor-core kernel does not take.  X and W are read in their stored type
// (float32 or bfloat16, widened exactly); products and sums are float32, never
// TF32.  Each output element is one thread's sum over k in ascending order, so
// a token's result does not depend on how many other tokens are in the call
// (the property the reference demands of its batched kernels,
// src/kernels.cu:2415-2454).  The reference's counterparts are the warp-per-row
// kernels `k_mv_*` / `k_mv_*_b` (src/kernels.cu:116-144, 534-549).
#include "common.cuh"

#define GS_BM 64
#define GS_BN 64
#define GS_BK 16

template <typename TX, typename TW, typename TO, bool ACCUM>
__global__ void __launch_bounds__(256)
k_gemm_simt(const TX* __restrict__ X, const TW* __restrict__ W, const float* __restrict__ bias,
            TO* __restrict__ out, int n, int n_out, int K, long long ldx, long long ldo) {
    __shared__ float Xs[GS_BK][GS_BM + 4];
    __shared__ float Ws[GS_BK][GS_BN + 4];
    int tid = threadIdx.x;
    int t0 = blockIdx.y * GS_BM, r0 = blockIdx.x * GS_BN;
    int ty = tid / 16, tx = tid % 16;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

    int lrow = tid / 4, lk = (tid % 4) * 4;
    for (int k0 = 0; k0 < K; k0 += GS_BK) {
#pragma unroll
        for (int q = 0; q < 4; q++) {
            int k = k0 + lk + q;
            int t = t0 + lrow, r = r0 + lrow;
            Xs[lk + q][lrow] = (t < n && k < K) ? xr_to_f32<TX>(X[(size_t)t * ldx + k]) : 0.f;
            Ws[lk + q][lrow] = (r < n_out && k < K) ? xr_to_f32<TW>(W[(size_t)r * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GS_BK; kk++) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = Xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int t = t0 + ty * 4 + i;
        if (t >= n) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int r = r0 + tx * 4 + j;
            if (r >= n_out) continue;
            float v = acc[i][j];
            if (bias) v += bias[r];
            size_t o = (size_t)t * ldo + r;
            if (ACCUM) out[o] = xr_from_f32<TO>(xr_to_f32<TO>(out[o]) + v);
            else out[o] = xr_from_f32<TO>(v);
        }
    }
}

template <typename TX, typename TW>
static int launch_simt(const void* X, const void* W, const float* bias, void* out, int out_dtype, int accumulate,
                       int n, int n_out, int K, long long ldx, long long ldo, cudaStream_t stream) {
    dim3 grid((n_out + GS_BN - 1) / GS_BN, (n + GS_BM - 1) / GS_BM);
    if (grid.y > 65535) return XR_ERR_ARG;
    if (accumulate) {
        if (out_dtype != XR_F32) return XR_ERR_ARG;
        k_gemm_simt<TX, TW, float, true><<<grid, 256, 0, stream>>>((const TX*)X, (const TW*)W, bias, (float*)out, n, n_out, K, ldx, ldo);
    } else if (out_dtype == XR_F32) {
        k_gemm_simt<TX, TW, float, false><<<grid, 256, 0, stream>>>((const TX*)X, (const TW*)W, bias, (float*)out, n, n_out, K, ldx, ldo);
    } else if (out_dtype == XR_BF16) {
        k_gemm_simt<TX, TW, __nv_bfloat16, false><<<grid, 256, 0, stream>>>((const TX*)X, (const TW*)W, bias, (__nv_bfloat16*)out, n, n_out, K, ldx, ldo);
    } else {
        return XR_ERR_ARG;
    }
    return xr_launch_status();
}

// X: [n, K] with row stride ldx; W: [n_out, K] dense; out: [n, n_out] with row stride ldo.
// accumulate != 0 adds into a float32 `out` (the residual stream).
XR_EXPORT int xr_gemm_simt(const void* X, int x_dtype, const void* W, int w_dtype, const float* bias, void* out,
                           int out_dtype, int accumulate, int n, int n_out, int K, long long ldx, long long ldo,
                           cudaStream_t stream) {
    if (n < 1 || n_out < 1 || K < 1 || ldx < K || ldo < n_out) return XR_ERR_ARG;
    if (x_dtype == XR_F32 && w_dtype == XR_F32) return launch_simt<float, float>(X, W, bias, out, out_dtype, accumulate, n, n_out, K, ldx, ldo, stream);
    if (x_dtype == XR_F32 && w_dtype == XR_BF16) return launch_simt<float, __nv_bfloat16>(X, W, bias, out, out_dtype, accumulate, n, n_out, K, ldx, ldo, stream);
    if (x_dtype == XR_BF16 && w_dtype == XR_F32) return launch_simt<__nv_bfloat16, float>(X, W, bias, out, out_dtype, accumulate, n, n_out, K, ldx, ldo, stream);
    if (x_dtype == XR_BF16 && w_dtype == XR_BF16) return launch_simt<__nv_bfloat16, __nv_bfloat16>(X, W, bias, out, out_dtype, accumulate, n, n_out, K, ldx, ldo, stream);
    return XR_ERR_ARG;
}
