// Causal attention over the paged cache on CUDA cores, float32 arithmetic:
// the attention of the true 32-bit path (and the checking twin of the
// tensor-core kernel).  One warp per (token, query head).  For the query at
// position p, head h, kv head h / (H/K):
//   s_t = (q . k_t) * scale   for t0 <= t <= p,  t0 = max(0, p - window + 1) (0 without a window)
//   a = softmax(s),  o = sum_t a_t v_t
// (src/model.c:3548-3589; softmax src/model.c:3409-3415).  Keys are taken in
// chunks of 32 in ascending order with a running maximum, so a query's result
// depends on its position and the keys only -- not on how the step was cut or
// what else is in the batch.  The reference's kernels are `k_attn`
// (src/kernels.cu:2043-2141) and the split `k_attn_dec` + `k_attn_merge`
// (src/kernels.cu:2171-2270).
//
// Every token's keys and values, its own included, are read from the cache:
// the store kernel runs before this one.
#include "common.cuh"
#include <math.h>

struct AttnArgs {
    const void* q;               // [n, q_row_stride] ; head h at offset h * hd
    void* out;                   // [n, H * hd]
    const void* cache_k;         // this layer's K block of page 0
    const int* positions;        // [n]
    const int* tok_seg;          // [n]
    const int* block_tables;     // [n_seg][max_pages]
    long long page_stride, v_offset, q_row_stride;
    int n, H, K, hd, max_pages, page_size, window;
    float scale;
};

#define AS_MAX_HD 256

template <typename T>
__global__ void __launch_bounds__(128)
k_attention_simt(AttnArgs a) {
    __shared__ float qs[4][AS_MAX_HD];
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    long long idx = (long long)blockIdx.x * 4 + warp;
    if (idx >= (long long)a.n * a.H) return;
    int t = (int)(idx / a.H), h = (int)(idx % a.H);
    int kvh = h / (a.H / a.K);
    int pos = a.positions[t];
    const int* bt = a.block_tables + (size_t)a.tok_seg[t] * a.max_pages;
    const T* qrow = (const T*)a.q + (size_t)t * a.q_row_stride + (size_t)h * a.hd;
    for (int i = lane; i < a.hd; i += 32) qs[warp][i] = xr_to_f32<T>(qrow[i]);
    __syncwarp();

    int t0 = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    const int ND = AS_MAX_HD / 32;
    float acc[ND];
#pragma unroll
    for (int i = 0; i < ND; i++) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    const T* kbase = (const T*)a.cache_k;

    for (int k0 = t0; k0 <= pos; k0 += 32) {
        int kp = k0 + lane;
        bool valid = kp <= pos;
        long long off = 0;
        float s = -INFINITY;
        if (valid) {
            int page = bt[kp / a.page_size];
            off = (long long)page * a.page_stride + ((long long)kvh * a.page_size + (kp % a.page_size)) * a.hd;
            const T* kr = kbase + off;
            float dot = 0.f;
            for (int i = 0; i < a.hd; i++) dot = fmaf(qs[warp][i], xr_to_f32<T>(kr[i]), dot);
            s = dot * a.scale;
        }
        float cm = xr_warp_max(s);
        float m_new = fmaxf(m, cm);
        float corr = expf(m - m_new);            // 0 on the first chunk (m = -inf)
        float p = valid ? expf(s - m_new) : 0.f;
        l = l * corr + xr_warp_sum(p);
#pragma unroll
        for (int i = 0; i < ND; i++) acc[i] *= corr;
        int cnt = min(32, pos - k0 + 1);
        for (int j = 0; j < cnt; j++) {
            float pj = __shfl_sync(0xffffffffu, p, j);
            long long oj = __shfl_sync(0xffffffffu, off, j);
            const T* vr = kbase + oj + a.v_offset;
#pragma unroll
            for (int i = 0; i < ND; i++) {
                int dd = lane + 32 * i;
                if (dd < a.hd) acc[i] = fmaf(pj, xr_to_f32<T>(vr[dd]), acc[i]);
            }
        }
        m = m_new;
    }
    T* orow = (T*)a.out + (size_t)t * a.H * a.hd + (size_t)h * a.hd;
    float inv = 1.0f / l;
#pragma unroll
    for (int i = 0; i < ND; i++) {
        int dd = lane + 32 * i;
        if (dd < a.hd) orow[dd] = xr_from_f32<T>(acc[i] * inv);
    }
}

XR_EXPORT int xr_attention_simt(const void* q, void* out, int dtype, const void* cache_k, const int* positions,
                                const int* tok_seg, const int* block_tables, long long page_stride,
                                long long v_offset, long long q_row_stride, int n, int H, int K, int hd,
                                int max_pages, int page_size, int window, float scale, cudaStream_t stream) {
    if (n < 1 || H < 1 || K < 1 || H % K != 0 || hd < 1 || hd > AS_MAX_HD || page_size < 1 || window < 0)
        return XR_ERR_ARG;
    AttnArgs a{q, out, cache_k, positions, tok_seg, block_tables, page_stride, v_offset, q_row_stride,
               n, H, K, hd, max_pages, page_size, window, scale};
    long long warps = (long long)n * H;
    long long blocks = (warps + 3) / 4;
    if (blocks > 0x7fffffffLL) return XR_ERR_ARG;
    if (dtype == XR_F32) k_attention_simt<float><<<(unsigned)blocks, 128, 0, stream>>>(a);
    else if (dtype == XR_BF16) k_attention_simt<__nv_bfloat16><<<(unsigned)blocks, 128, 0, stream>>>(a);
    else return XR_ERR_ARG;
    return xr_launch_status();
}
