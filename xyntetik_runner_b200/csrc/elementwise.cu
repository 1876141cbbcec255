// Memory-bound kernels of the step: embedding gather, RMSNorm, rotation + paged
// key/value store, SwiGLU.  The residual stream is float32 in both precisions;
// "activation dtype" below is what matrix products read and write (bfloat16 in
// the serving path, float32 in the true 32-bit path).
#include "common.cuh"

// ---------------------------------------------------------------------------
// Embedding: x[t] = E[id_t], ids outside [0, vocab) read row 0
// (the reference does the same on the host, src/model.c:6148-6162).
// ---------------------------------------------------------------------------
// `feed` (optional): ids[t] = -(1 + j) stands for feed[j], a token that an earlier step of the same stream left
// on the device (the one it sampled), so that the host need not have seen it when it describes this step.
template <typename TW>
__global__ void k_embed(const TW* __restrict__ table, const int* __restrict__ ids, const int* __restrict__ feed,
                        float* __restrict__ x, int d, int vocab, int n_feed) {
    xr_pdl_launch();
    // The token ids are part of the step's description and the table is a weight: the row is read before the kernel
    // ahead is complete, sixteen values a thread in one run of loads; only the stores wait.  (A fed token is another
    // matter: it is what the step before sampled, so it is read after the wait.)
    int t = blockIdx.x;
    int id = ids[t];
    const bool fed = feed != nullptr && id < 0 && -(id + 1) < n_feed;
    if (fed) {
        xr_pdl_wait();
        id = feed[-(id + 1)];
    }
    if (id < 0 || id >= vocab) id = 0;
    const TW* row = table + (size_t)id * d;
    float* out = x + (size_t)t * d;
    for (int i0 = threadIdx.x; i0 < d; i0 += 16 * blockDim.x) {
        TW v[16];
#pragma unroll
        for (int k = 0; k < 16; k++) {
            int i = i0 + k * blockDim.x;
            v[k] = row[i < d ? i : d - 1];
        }
        if (i0 == (int)threadIdx.x && !fed) xr_pdl_wait();
#pragma unroll
        for (int k = 0; k < 16; k++) {
            int i = i0 + k * blockDim.x;
            if (i < d) out[i] = xr_to_f32<TW>(v[k]);
        }
    }
}

XR_EXPORT int xr_embed(const void* table, int table_dtype, const int* ids, const int* feed, int n_feed, float* x, int n, int d,
                       int vocab, cudaStream_t stream) {
    if (n < 1 || d < 1 || vocab < 1 || n_feed < 0) return XR_ERR_ARG;
    if (table_dtype == XR_F32) xr_launch((k_embed<float>), dim3(n), dim3(256), 0, stream, (const float*)table, ids, feed, x, d, vocab, n_feed);
    else if (table_dtype == XR_BF16) xr_launch((k_embed<__nv_bfloat16>), dim3(n), dim3(256), 0, stream, (const __nv_bfloat16*)table, ids, feed, x, d, vocab, n_feed);
    else return XR_ERR_ARG;
    return xr_launch_status();
}

// ---------------------------------------------------------------------------
// RMSNorm of float32 rows: y = x * rsqrt(mean(x^2) + eps) * w
// (src/model.c:3386-3392; the reference's kernel is src/kernels.cu:32-48).
// `rows` (optional) picks the rows to normalise: out[i] = norm(x[rows[i]]).
// One block per row; the reduction order depends on the width only.
// ---------------------------------------------------------------------------
template <typename TO>
__global__ void k_rmsnorm(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ w,
                          TO* __restrict__ out, int d, float eps) {
    xr_pdl_launch();
    xr_pdl_wait();
    __shared__ float scratch[33];
    int r = rows ? rows[blockIdx.x] : blockIdx.x;
    const float* xr = x + (size_t)r * d;
    TO* o = out + (size_t)blockIdx.x * d;
    constexpr int PER = 16;                     // elements a thread can keep: rows up to 16 * blockDim.x stay in registers
    if (d <= PER * (int)blockDim.x) {
        float v[PER];
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < PER; k++) {
            int i = threadIdx.x + k * blockDim.x;
            v[k] = i < d ? xr[i] : 0.f;
            ss += v[k] * v[k];
        }
        ss = xr_block_sum(ss, scratch);
        float scale = 1.0f / sqrtf(ss / (float)d + eps);
#pragma unroll
        for (int k = 0; k < PER; k++) {
            int i = threadIdx.x + k * blockDim.x;
            if (i < d) o[i] = xr_from_f32<TO>(v[k] * scale * w[i]);
        }
        return;
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) { float v = xr[i]; ss += v * v; }
    ss = xr_block_sum(ss, scratch);
    float scale = 1.0f / sqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = xr_from_f32<TO>(xr[i] * scale * w[i]);
}

// Rows whose width is a multiple of four: a thread keeps up to eight float4 of the row, so a row needs few
// threads (width / 32) and many rows are in flight on an SM at once.  The block size, and with it the order
// of the sum, is a function of the width alone.
__device__ __forceinline__ void rms_store4(float* o, float4 v) { *reinterpret_cast<float4*>(o) = v; }
__device__ __forceinline__ void rms_store4(__nv_bfloat16* o, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&a); u.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(o) = u;
}
template <typename TO>
__global__ void k_rmsnorm_vec(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ w,
                              TO* __restrict__ out, int d, float eps) {
    xr_pdl_launch();
    xr_pdl_wait();
    __shared__ float scratch[33];
    constexpr int PER = 8;
    const int r = rows ? rows[blockIdx.x] : blockIdx.x;
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)r * d);
    const float4* w4 = reinterpret_cast<const float4*>(w);
    TO* o = out + (size_t)blockIdx.x * d;
    const int quads = d >> 2;
    float4 v[PER];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < PER; k++) {
        int i = threadIdx.x + k * blockDim.x;
        v[k] = i < quads ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int k = 0; k < PER; k++) ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    ss = xr_block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
#pragma unroll
    for (int k = 0; k < PER; k++) {
        int i = threadIdx.x + k * blockDim.x;
        if (i < quads) {
            float4 g = w4[i];
            rms_store4(o + 4 * (size_t)i, make_float4(v[k].x * scale * g.x, v[k].y * scale * g.y, v[k].z * scale * g.z, v[k].w * scale * g.w));
        }
    }
}

XR_EXPORT int xr_rmsnorm(const float* x, const int* rows, const float* w, void* out, int out_dtype, int n, int d,
                         float eps, cudaStream_t stream) {
    if (n < 1 || d < 1) return XR_ERR_ARG;
    if (out_dtype != XR_F32 && out_dtype != XR_BF16) return XR_ERR_ARG;
    if ((d & 3) == 0 && d <= 32 * 1024 && (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) == 0) {
        int threads = (((d / 4 + 7) / 8 + 31) / 32) * 32;          // eight float4 per thread cover the row
        if (out_dtype == XR_F32) xr_launch((k_rmsnorm_vec<float>), dim3(n), dim3(threads), 0, stream, x, rows, w, (float*)out, d, eps);
        else xr_launch((k_rmsnorm_vec<__nv_bfloat16>), dim3(n), dim3(threads), 0, stream, x, rows, w, (__nv_bfloat16*)out, d, eps);
        return xr_launch_status();
    }
    int threads = d >= 2048 ? 512 : 256;
    if (out_dtype == XR_F32) xr_launch((k_rmsnorm<float>), dim3(n), dim3(threads), 0, stream, x, rows, w, (float*)out, d, eps);
    else if (out_dtype == XR_BF16) xr_launch((k_rmsnorm<__nv_bfloat16>), dim3(n), dim3(threads), 0, stream, x, rows, w, (__nv_bfloat16*)out, d, eps);
    else return XR_ERR_ARG;
    return xr_launch_status();
}

// ---------------------------------------------------------------------------
// Rotation of Q and K and the store of K, V into their pages.
//
// qkv: [n, (H + 2K) * hd] rows as the fused projection wrote them (Q heads,
// then K heads, then V heads).  For the token at position p and pair index
// j < rotary_dim/2: a = p * inv_freq[j] in float32, then
// (x0, x1) -> (x0 c - x1 s, x0 s + x1 c) on elements (j, j + rotary_dim/2)
// (src/model.c:3514-3532, the half-split pairing).  Q is rotated in place; K
// is rotated and written to the cache, V copied (src/model.c:6276-6310).
// The cache of a layer group is [page][layer][K|V][kv head][token in page][hd];
// `cache_k` points at this layer's K block of page 0.
// ---------------------------------------------------------------------------
struct RopeStoreArgs {
    void* qkv;
    const int* positions;
    const int* tok_seg;
    const int* block_tables;     // [n_seg][max_pages]
    const float* inv_freq;       // [rotary_dim / 2] or null when rotary_dim == 0
    void* cache_k;               // null: this layer stores nothing (it reads another layer's cache)
    long long page_stride;       // elements between pages
    long long v_offset;          // elements from a layer's K block to its V block
    int n, H, K, hd, rotary_dim, max_pages, page_size;
    int adjacent;                // 0: pair j is elements (j, j + rotary_dim/2); 1: elements (2j, 2j + 1)
    float mscale;                // factor on the cosines and sines (1 unless the position encoding scales magnitudes)
};

// One block per token.  A thread owns pair index j (and every `blockDim.x / half`-th head): the angle
// pos * inv_freq[j] and its cosine and sine are computed once and used for all the Q and K heads.
template <typename T>
__global__ void k_rope_store(RopeStoreArgs a) {
    xr_pdl_launch();
    xr_pdl_wait();
    const int t = blockIdx.x;
    const int qkv_dim = (a.H + 2 * a.K) * a.hd;
    T* row = (T*)a.qkv + (size_t)t * qkv_dim;
    const int pos = a.positions[t];
    const int half = a.rotary_dim >> 1;
    T* kdst = nullptr;
    if (a.cache_k != nullptr) {
        int page = a.block_tables[(size_t)a.tok_seg[t] * a.max_pages + pos / a.page_size];
        kdst = (T*)a.cache_k + (size_t)page * a.page_stride + (size_t)(pos % a.page_size) * a.hd;
    }
    const size_t head_step = (size_t)a.page_size * a.hd;          // between kv heads inside a page
    // rotated pairs of the Q and K heads
    if (half > 0) {
        const int lanes = blockDim.x / half > 0 ? blockDim.x / half : 1;      // heads handled side by side
        const int j = threadIdx.x % half, h0 = threadIdx.x / half;
        if (threadIdx.x < lanes * half) {
            float ang = (float)pos * a.inv_freq[j];
            float c = cosf(ang) * a.mscale, s = sinf(ang) * a.mscale;
            const int i0 = a.adjacent ? 2 * j : j, i1 = a.adjacent ? 2 * j + 1 : j + half;
            for (int head = h0; head < a.H + a.K; head += lanes) {
                T* src = row + (size_t)head * a.hd;
                float x0 = xr_to_f32<T>(src[i0]), x1 = xr_to_f32<T>(src[i1]);
                T y0 = xr_from_f32<T>(x0 * c - x1 * s), y1 = xr_from_f32<T>(x0 * s + x1 * c);
                if (head < a.H) { src[i0] = y0; src[i1] = y1; }
                else if (kdst) { T* d = kdst + (size_t)(head - a.H) * head_step; d[i0] = y0; d[i1] = y1; }
            }
        }
    }
    if (kdst == nullptr) return;
    // the part of K beyond the rotated dimensions, and V, are copied
    const int tail = a.hd - 2 * half;
    for (int i = threadIdx.x; i < a.K * tail; i += blockDim.x) {
        int kvh = i / tail, e = 2 * half + i % tail;
        kdst[(size_t)kvh * head_step + e] = row[(size_t)(a.H + kvh) * a.hd + e];
    }
    T* vdst = kdst + a.v_offset;
    for (int i = threadIdx.x; i < a.K * a.hd; i += blockDim.x) {
        int kvh = i / a.hd, e = i % a.hd;
        vdst[(size_t)kvh * head_step + e] = row[(size_t)(a.H + a.K + kvh) * a.hd + e];
    }
}

// bfloat16 rows whose head size and rotated width are multiples of eight and sixteen: every access is a
// 16-byte vector of eight elements.  The cosines and sines of the token's angles are computed once, in
// shared memory; a thread then takes (head, group of eight pairs) units.
struct __align__(16) Bf16x8 { __nv_bfloat162 p[4]; };
__global__ void __launch_bounds__(256)
k_rope_store_vec(RopeStoreArgs a) {
    xr_pdl_launch();
    // positions, block tables and frequencies do not change while the step runs: the token's page and the table of
    // its angles are worked out before the kernel ahead (the product that writes the rows) is complete
    extern __shared__ float rope_cs[];                 // [half] cosines, [half] sines
    const int t = blockIdx.x;
    const int qkv_dim = (a.H + 2 * a.K) * a.hd;
    __nv_bfloat16* row = (__nv_bfloat16*)a.qkv + (size_t)t * qkv_dim;
    const int pos = a.positions[t];
    const int half = a.rotary_dim >> 1;
    __nv_bfloat16* kdst = nullptr;
    if (a.cache_k != nullptr) {
        int page = a.block_tables[(size_t)a.tok_seg[t] * a.max_pages + pos / a.page_size];
        kdst = (__nv_bfloat16*)a.cache_k + (size_t)page * a.page_stride + (size_t)(pos % a.page_size) * a.hd;
    }
    const size_t head_step = (size_t)a.page_size * a.hd;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        float ang = (float)pos * a.inv_freq[j];
        rope_cs[j] = cosf(ang) * a.mscale;
        rope_cs[half + j] = sinf(ang) * a.mscale;
    }
    __syncthreads();
    xr_pdl_wait();
    const int groups = half >> 3;                      // groups of eight pairs per head
    const int rot_heads = kdst ? a.H + a.K : a.H;      // without a cache to write, K is not needed
    for (int u = threadIdx.x; u < rot_heads * groups; u += blockDim.x) {
        int head = u / groups, j0 = (u % groups) << 3;
        if (a.adjacent) {
            // eight pairs are sixteen consecutive elements: two vectors, each bfloat162 one pair
            __nv_bfloat16* src = row + (size_t)head * a.hd + 2 * j0;
            Bf16x8 v[2] = {*reinterpret_cast<const Bf16x8*>(src), *reinterpret_cast<const Bf16x8*>(src + 8)};
#pragma unroll
            for (int k = 0; k < 8; k++) {
                float2 x = __bfloat1622float2(v[k >> 2].p[k & 3]);
                float c = rope_cs[j0 + k], sn = rope_cs[half + j0 + k];
                v[k >> 2].p[k & 3] = __floats2bfloat162_rn(x.x * c - x.y * sn, x.x * sn + x.y * c);
            }
            __nv_bfloat16* dst = head < a.H ? src : kdst + (size_t)(head - a.H) * head_step + 2 * j0;
            *reinterpret_cast<Bf16x8*>(dst) = v[0];
            *reinterpret_cast<Bf16x8*>(dst + 8) = v[1];
            continue;
        }
        __nv_bfloat16* src = row + (size_t)head * a.hd + j0;
        Bf16x8 lo = *reinterpret_cast<const Bf16x8*>(src), hi = *reinterpret_cast<const Bf16x8*>(src + half);
#pragma unroll
        for (int k = 0; k < 4; k++) {
            float2 x0 = __bfloat1622float2(lo.p[k]), x1 = __bfloat1622float2(hi.p[k]);
            float c0 = rope_cs[j0 + 2 * k], c1 = rope_cs[j0 + 2 * k + 1];
            float s0 = rope_cs[half + j0 + 2 * k], s1 = rope_cs[half + j0 + 2 * k + 1];
            lo.p[k] = __floats2bfloat162_rn(x0.x * c0 - x1.x * s0, x0.y * c1 - x1.y * s1);
            hi.p[k] = __floats2bfloat162_rn(x0.x * s0 + x1.x * c0, x0.y * s1 + x1.y * c1);
        }
        __nv_bfloat16* dst = head < a.H ? src : kdst + (size_t)(head - a.H) * head_step + j0;
        *reinterpret_cast<Bf16x8*>(dst) = lo;
        *reinterpret_cast<Bf16x8*>(dst + half) = hi;
    }
    if (kdst == nullptr) return;
    const int tail8 = (a.hd - 2 * half) >> 3, hd8 = a.hd >> 3;
    for (int i = threadIdx.x; i < a.K * tail8; i += blockDim.x) {
        int kvh = i / tail8, e = 2 * half + ((i % tail8) << 3);
        *reinterpret_cast<Bf16x8*>(kdst + (size_t)kvh * head_step + e) = *reinterpret_cast<const Bf16x8*>(row + (size_t)(a.H + kvh) * a.hd + e);
    }
    __nv_bfloat16* vdst = kdst + a.v_offset;
    for (int i = threadIdx.x; i < a.K * hd8; i += blockDim.x) {
        int kvh = i / hd8, e = (i % hd8) << 3;
        *reinterpret_cast<Bf16x8*>(vdst + (size_t)kvh * head_step + e) = *reinterpret_cast<const Bf16x8*>(row + (size_t)(a.H + a.K + kvh) * a.hd + e);
    }
}

XR_EXPORT int xr_rope_store(void* qkv, int dtype, const int* positions, const int* tok_seg, const int* block_tables,
                            const float* inv_freq, void* cache_k, long long page_stride, long long v_offset,
                            int n, int H, int K, int hd, int rotary_dim, int max_pages, int page_size,
                            int adjacent_pairs, float mscale, cudaStream_t stream) {
    if (n < 1 || H < 1 || K < 1 || hd < 1 || rotary_dim < 0 || rotary_dim > hd || (rotary_dim & 1) ||
        page_size < 1 || H + 2 * K > 65535)
        return XR_ERR_ARG;
    RopeStoreArgs a{qkv, positions, tok_seg, block_tables, inv_freq, cache_k, page_stride, v_offset,
                    n, H, K, hd, rotary_dim, max_pages, page_size, adjacent_pairs ? 1 : 0, mscale};
    int threads = 256;
    if (dtype == XR_BF16 && (hd & 7) == 0 && (rotary_dim & 15) == 0 && ((uintptr_t)qkv & 15) == 0 &&
        (cache_k == nullptr || ((((uintptr_t)cache_k) & 15) == 0 && (page_stride & 7) == 0 && (v_offset & 7) == 0))) {
        xr_launch(k_rope_store_vec, dim3(n), dim3(threads), (size_t)rotary_dim * sizeof(float), stream, a);
        return xr_launch_status();
    }
    if (dtype == XR_F32) xr_launch((k_rope_store<float>), dim3(n), dim3(threads), 0, stream, a);
    else if (dtype == XR_BF16) xr_launch((k_rope_store<__nv_bfloat16>), dim3(n), dim3(threads), 0, stream, a);
    else return XR_ERR_ARG;
    return xr_launch_status();
}

// ---------------------------------------------------------------------------
// Activation of a feed-forward: gated, h = act(g) * u with g, u the two halves of each row of gu [n, 2F]
// (src/model.c:4425-4452, `gated_act`); ungated, h = act(x) of x [n, F] (src/model.c:6380-6396).
// act 1: SiLU, g / (1 + exp(-g)), 0 for g < -80 (src/model.c:4451-4452; the reference's kernel is
// src/kernels.cu:2868-2874); act 2: tanh-GELU, 0.5 g (1 + tanh(0.7978845608 (g + 0.044715 g^3)))
// (src/model.c:4438-4441); act 0: none.  Full-precision expf and tanhf: this is the kernel of the true 32-bit path.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float xr_activation(int act, float g) {
    if (act == 1) return g < -80.0f ? 0.0f : g / (1.0f + expf(-g));
    if (act == 2) return 0.5f * g * (1.0f + tanhf(0.7978845608f * (g + 0.044715f * g * g * g)));
    return g;
}

template <typename T>
__global__ void k_act_mul(const T* gu, T* h, int n, int F, int act, int gated) {       // (h may be gu: no __restrict__)
    xr_pdl_launch();
    xr_pdl_wait();
    size_t total = (size_t)n * F;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        size_t t = i / F, f = i % F;
        float v;
        if (gated) v = xr_activation(act, xr_to_f32<T>(gu[t * 2 * F + f])) * xr_to_f32<T>(gu[t * 2 * F + F + f]);
        else v = xr_activation(act, xr_to_f32<T>(gu[i]));
        h[i] = xr_from_f32<T>(v);
    }
}

// gated: gu [n, 2F] -> h [n, F]; ungated: gu [n, F] -> h [n, F] (h may be gu)
XR_EXPORT int xr_act_mul(const void* gu, void* h, int dtype, int n, int F, int act, int gated, cudaStream_t stream) {
    if (n < 1 || F < 1 || act < 0 || act > 2) return XR_ERR_ARG;
    size_t total = (size_t)n * F;
    int blocks = (int)((total + 255) / 256 < (size_t)xr_sm_count() * 16 ? (total + 255) / 256 : xr_sm_count() * 16);
    if (dtype == XR_F32) xr_launch((k_act_mul<float>), dim3(blocks), dim3(256), 0, stream, (const float*)gu, (float*)h, n, F, act, gated);
    else if (dtype == XR_BF16) xr_launch((k_act_mul<__nv_bfloat16>), dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)h, n, F, act, gated);
    else return XR_ERR_ARG;
    return xr_launch_status();
}

// ---------------------------------------------------------------------------
// y[t][i] += d[t][i] on the float32 residual stream (src/kernels.cu:2903-2906),
// for parts whose last product cannot add into the stream itself.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void k_residual_add(float* __restrict__ x, const T* __restrict__ dlt, size_t total) {
    xr_pdl_launch();
    xr_pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        x[i] += xr_to_f32<T>(dlt[i]);
}

XR_EXPORT int xr_residual_add(float* x, const void* dlt, int dtype, int n, int d, cudaStream_t stream) {
    if (n < 1 || d < 1) return XR_ERR_ARG;
    size_t total = (size_t)n * d;
    int blocks = (int)((total + 255) / 256 < xr_sm_count() * 16 ? (total + 255) / 256 : xr_sm_count() * 16);
    if (dtype == XR_F32) xr_launch((k_residual_add<float>), dim3(blocks), dim3(256), 0, stream, x, (const float*)dlt, total);
    else if (dtype == XR_BF16) xr_launch((k_residual_add<__nv_bfloat16>), dim3(blocks), dim3(256), 0, stream, x, (const __nv_bfloat16*)dlt, total);
    else return XR_ERR_ARG;
    return xr_launch_status();
}

#ifdef XR_TRACE
// ---------------------------------------------------------------------------
// Tracing build only: the records of all source files, one after another.
// host: [files][4096][4] (time resident, time the wait returned, grid packed 20 bits a dimension, block size);
// counts: [files] records written since the last call.  Returns the number of files.
// ---------------------------------------------------------------------------
static xr_tr_dump_fn g_tr_fns[32];
static int g_tr_nfns = 0;
extern "C" int xr_trace_add(xr_tr_dump_fn fn) { if (g_tr_nfns < 32) g_tr_fns[g_tr_nfns++] = fn; return g_tr_nfns; }
XR_EXPORT int xr_trace_dump(unsigned long long* host, unsigned int* counts) {
    for (int i = 0; i < g_tr_nfns; i++) g_tr_fns[i](host + (size_t)i * 4096 * 4, counts + i);
    return g_tr_nfns;
}
#endif
