// Kernels that finish a split-K product and do the next memory-bound op in the same pass, so that a decode
// step does not pay a launch and a round trip through memory for each:
//   * sum of partials (+ bias) -> added into the float32 residual stream -> RMSNorm of the new row
//     (the reference runs `k_add` src/kernels.cu:2903 and `k_rmsnorm` :32 as two kernels after its matvec);
//   * sum of partials (+ bias) of the fused QKV product -> rotation of Q and K -> Q to the activation
//     buffer, K and V into their pages (`k_rope`, `k_store_kv`, src/kernels.cu:1918, 2008).
// Partials are [splits][n][width] float32 and are summed in split order, so the result is deterministic.
#include "common.cuh"

// One block per token.  A thread owns up to FIN_PER elements of the row (strided by the block size) and keeps
// them in registers; the partial sums are read with all of a thread's loads of one split in flight together
// (the splits are summed in order, so the result does not depend on timing).
#define FIN_PER 8
template <typename TO>
__global__ void __launch_bounds__(1024)
k_finish_add_rmsnorm(const float* __restrict__ partial, int splits, int n, const float* __restrict__ bias,
                     float* __restrict__ x, const float* __restrict__ w, TO* __restrict__ out, int d, float eps) {
    xr_pdl_launch();
    xr_pdl_wait();
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    float* xr = x + (size_t)t * d;
    TO* o = out + (size_t)t * d;
    float ss = 0.f;
    if (d <= FIN_PER * (int)blockDim.x) {
        float acc[FIN_PER];
#pragma unroll
        for (int k = 0; k < FIN_PER; k++) acc[k] = 0.f;
        const float* p = partial + (size_t)t * d + threadIdx.x;
        const size_t split_stride = (size_t)n * d;
#pragma unroll 4
        for (int s = 0; s < splits; s++) {
            float v[FIN_PER];
#pragma unroll
            for (int k = 0; k < FIN_PER; k++) v[k] = (int)(threadIdx.x + k * blockDim.x) < d ? __ldcg(p + (size_t)s * split_stride + k * blockDim.x) : 0.f;
#pragma unroll
            for (int k = 0; k < FIN_PER; k++) acc[k] += v[k];
        }
#pragma unroll
        for (int k = 0; k < FIN_PER; k++) {
            int i = threadIdx.x + k * blockDim.x;
            if (i < d) {
                float v = acc[k];
                if (bias) v += bias[i];
                v = xr[i] + v;
                xr[i] = v;
                acc[k] = v;
                ss += v * v;
            }
        }
        ss = xr_block_sum(ss, scratch);
        float scale = 1.0f / sqrtf(ss / (float)d + eps);
#pragma unroll
        for (int k = 0; k < FIN_PER; k++) {
            int i = threadIdx.x + k * blockDim.x;
            if (i < d) o[i] = xr_from_f32<TO>(acc[k] * scale * w[i]);
        }
        return;
    }
    // rows too wide for the registers: two passes through global memory
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = 0.f;
        for (int s = 0; s < splits; s++) v += partial[((size_t)s * n + t) * d + i];
        if (bias) v += bias[i];
        v = xr[i] + v;
        xr[i] = v;
        ss += v * v;
    }
    ss = xr_block_sum(ss, scratch);
    float scale = 1.0f / sqrtf(ss / (float)d + eps);
    __syncthreads();
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = xr_from_f32<TO>(xr[i] * scale * w[i]);
}

// The same for few tokens: a cluster of FIN_CLUSTER blocks per token, each block owning a contiguous slice of
// the row, so that the partial sums are read by eight times as many threads.  The slices' sums of squares
// meet through distributed shared memory (each block writes its own into all eight) and every block adds them
// in rank order.
#define FIN_CLUSTER 8
#define FIN_CL_PER 4
__device__ __forceinline__ uint32_t fin_cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void fin_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// writes `v` to the same variable in the shared memory of block `rank` of the cluster
__device__ __forceinline__ void fin_cluster_write(float* mine, uint32_t rank, float v) {
    uint32_t local = (uint32_t)__cvta_generic_to_shared(mine), remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

template <typename TO, int PER>
__global__ void __launch_bounds__(256)
k_finish_add_rmsnorm_cluster(const float* __restrict__ partial, int splits, int n, const float* __restrict__ bias,
                             float* __restrict__ x, const float* __restrict__ w, TO* __restrict__ out, int d, int slice, float eps) {
    xr_pdl_launch();
    // "this block runs": its neighbours wait for that before they write into its shared memory
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    __shared__ float scratch[33];
    __shared__ float slice_ss[FIN_CLUSTER];      // every block's sum of squares, written here by that block
    const int t = blockIdx.x / FIN_CLUSTER;
    const int rank = (int)fin_cluster_rank();
    const int c0 = rank * slice, c1 = min(d, c0 + slice);          // slice <= PER * blockDim.x
    float* xr = x + (size_t)t * d;
    TO* o = out + (size_t)t * d;
    // Every load is unconditional (an index past the slice is clamped into it and its value dropped), so that all of
    // them are in flight at once.  The norm's weights and the bias are constants: they are read before the kernel
    // ahead is known to be complete; the residual and the partial sums after.
    int idx[PER];
    float wv[PER], bv[PER];
#pragma unroll
    for (int k = 0; k < PER; k++) {
        int i = c0 + threadIdx.x + k * blockDim.x;
        idx[k] = i < c1 ? i : c1 - 1;
        wv[k] = w[idx[k]];
        bv[k] = bias ? bias[idx[k]] : 0.f;
    }
    xr_pdl_wait();
    const size_t split_stride = (size_t)n * d;
    const float* p = partial + (size_t)t * d;
    float acc[PER], old[PER];
#pragma unroll
    for (int k = 0; k < PER; k++) { acc[k] = 0.f; old[k] = xr_ld_now(xr + idx[k]); }
    for (int s0 = 0; s0 < splits; s0 += 16) {
        float v[16][PER];
#pragma unroll
        for (int q = 0; q < 16; q++) {
            const float* ps = p + (size_t)min(s0 + q, splits - 1) * split_stride;
#pragma unroll
            for (int k = 0; k < PER; k++) v[q][k] = xr_ld_now(ps + idx[k]);
        }
        // nothing below may be scheduled among the loads above
#pragma unroll
        for (int q = 0; q < 16; q++)
#pragma unroll
            for (int k = 0; k < PER; k++) xr_ld_fence(v[q][k]);
#pragma unroll
        for (int q = 0; q < 16; q++) {
            const bool live = s0 + q < splits;
#pragma unroll
            for (int k = 0; k < PER; k++) acc[k] += live ? v[q][k] : 0.f;
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < PER; k++) {
        int i = c0 + threadIdx.x + k * blockDim.x;
        if (i < c1) {
            float v = old[k] + (acc[k] + bv[k]);
            xr[i] = v;
            acc[k] = v;
            ss += v * v;
        }
    }
    ss = xr_block_sum(ss, scratch);
    // each block hands its sum to all eight (itself included); after the one barrier nobody touches a neighbour's
    // shared memory again, so blocks may leave as they finish
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");      // (long since complete: all eight began together)
    if (threadIdx.x < FIN_CLUSTER) fin_cluster_write(&slice_ss[rank], (uint32_t)threadIdx.x, ss);
    fin_cluster_sync();
    float total = 0.f;
#pragma unroll
    for (int r = 0; r < FIN_CLUSTER; r++) total += slice_ss[r];
    float scale = 1.0f / sqrtf(total / (float)d + eps);
#pragma unroll
    for (int k = 0; k < PER; k++) {
        int i = c0 + threadIdx.x + k * blockDim.x;
        if (i < c1) o[i] = xr_from_f32<TO>(acc[k] * scale * wv[k]);
    }
}

// The same for more tokens than a latency-bound launch is worth tuning for (a decode step of 17 to a few hundred
// requests): one block per token, a thread owns four neighbouring elements and reads them as one 16-byte vector per
// split, so that the kernel issues a sixth of the instructions of the scalar versions (which, at 64 tokens, were bound
// by instruction issue: 8.9 us, issue slots 47 % busy for 10 MB of reads).  Same sums in the same order.
#define FIN_V4_PER 2                    // float4 a thread keeps: rows up to 8 * blockDim.x elements
__device__ __forceinline__ void fin_store4(float* o, float4 v) { *reinterpret_cast<float4*>(o) = v; }
__device__ __forceinline__ void fin_store4(__nv_bfloat16* o, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&a); u.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(o) = u;
}
template <typename TO>
__global__ void __launch_bounds__(1024)
k_finish_add_rmsnorm_vec4(const float* __restrict__ partial, int splits, int n, const float* __restrict__ bias,
                          float* __restrict__ x, const float* __restrict__ w, TO* __restrict__ out, int d, float eps) {
    xr_pdl_launch();
    __shared__ float scratch[33];
    const int t = blockIdx.x, quads = d >> 2;
    float4* xr = reinterpret_cast<float4*>(x + (size_t)t * d);
    TO* o = out + (size_t)t * d;
    // constants first (norm weights, bias), before the kernel ahead is known to be complete
    float4 wv[FIN_V4_PER], bv[FIN_V4_PER];
#pragma unroll
    for (int k = 0; k < FIN_V4_PER; k++) {
        const int i = threadIdx.x + k * blockDim.x;
        const int ic = i < quads ? i : quads - 1;
        wv[k] = reinterpret_cast<const float4*>(w)[ic];
        bv[k] = bias ? reinterpret_cast<const float4*>(bias)[ic] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    xr_pdl_wait();
    const size_t split_stride = ((size_t)n * d) >> 2;
    const float4* p = reinterpret_cast<const float4*>(partial) + (((size_t)t * d) >> 2);
    float4 acc[FIN_V4_PER];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < FIN_V4_PER; k++) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i >= quads) { acc[k] = make_float4(0.f, 0.f, 0.f, 0.f); continue; }
        float4 old = xr_ld_now4(xr + i);
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s0 = 0; s0 < splits; s0 += 8) {
            float4 v[8];
#pragma unroll
            for (int q = 0; q < 8; q++) v[q] = xr_ld_now4(p + (size_t)min(s0 + q, splits - 1) * split_stride + i);
#pragma unroll
            for (int q = 0; q < 8; q++) xr_ld_fence(v[q]);
#pragma unroll
            for (int q = 0; q < 8; q++)
                if (s0 + q < splits) { a.x += v[q].x; a.y += v[q].y; a.z += v[q].z; a.w += v[q].w; }
        }
        xr_ld_fence(old);
        a = make_float4(old.x + (a.x + bv[k].x), old.y + (a.y + bv[k].y), old.z + (a.z + bv[k].z), old.w + (a.w + bv[k].w));
        xr[i] = a;
        acc[k] = a;
        ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
    ss = xr_block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
#pragma unroll
    for (int k = 0; k < FIN_V4_PER; k++) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < quads)
            fin_store4(o + 4 * (size_t)i, make_float4(acc[k].x * scale * wv[k].x, acc[k].y * scale * wv[k].y,
                                                       acc[k].z * scale * wv[k].z, acc[k].w * scale * wv[k].w));
    }
}

// The cluster kernel with 16-byte vectors: a block's slice of the row is a multiple of four elements and a thread
// owns ONE quadruple of it, so a thread issues a dozen loads instead of several dozen and the kernel is bound by the
// trip to L2, not by instruction issue, also at 64 tokens.
template <typename TO>
__global__ void __launch_bounds__(256)
k_finish_add_rmsnorm_cluster4(const float* __restrict__ partial, int splits, int n, const float* __restrict__ bias,
                              float* __restrict__ x, const float* __restrict__ w, TO* __restrict__ out, int d, int slice, float eps) {
    xr_pdl_launch();
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");      // "this block runs"
    __shared__ float scratch[33];
    __shared__ float slice_ss[FIN_CLUSTER];
    const int t = blockIdx.x / FIN_CLUSTER;
    const int rank = (int)fin_cluster_rank();
    const int c0 = rank * slice, c1 = min(d, c0 + slice);                        // both multiples of four
    const int i = c0 + 4 * (int)threadIdx.x;                                     // this thread's quadruple
    const bool mine = i < c1;
    const int ic = mine ? i : c0;                                                // (clamped: every load is unconditional)
    float* xr = x + (size_t)t * d;
    const float4 wv = *reinterpret_cast<const float4*>(w + ic);
    const float4 bv = bias ? *reinterpret_cast<const float4*>(bias + ic) : make_float4(0.f, 0.f, 0.f, 0.f);
    xr_pdl_wait();
    const size_t split_stride = (size_t)n * d;
    const float* p = partial + (size_t)t * d + ic;
    float4 old = xr_ld_now4(reinterpret_cast<const float4*>(xr + ic));
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < splits; s0 += 16) {
        float4 v[16];
#pragma unroll
        for (int q = 0; q < 16; q++) v[q] = xr_ld_now4(reinterpret_cast<const float4*>(p + (size_t)min(s0 + q, splits - 1) * split_stride));
#pragma unroll
        for (int q = 0; q < 16; q++) xr_ld_fence(v[q]);
#pragma unroll
        for (int q = 0; q < 16; q++) {
            const bool live = s0 + q < splits;
            a.x += live ? v[q].x : 0.f; a.y += live ? v[q].y : 0.f; a.z += live ? v[q].z : 0.f; a.w += live ? v[q].w : 0.f;
        }
    }
    xr_ld_fence(old);
    a = make_float4(old.x + (a.x + bv.x), old.y + (a.y + bv.y), old.z + (a.z + bv.z), old.w + (a.w + bv.w));
    float ss = 0.f;
    if (mine) {
        *reinterpret_cast<float4*>(xr + i) = a;
        ss = a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
    ss = xr_block_sum(ss, scratch);
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (threadIdx.x < FIN_CLUSTER) fin_cluster_write(&slice_ss[rank], (uint32_t)threadIdx.x, ss);
    fin_cluster_sync();
    float total = 0.f;
#pragma unroll
    for (int r = 0; r < FIN_CLUSTER; r++) total += slice_ss[r];
    const float scale = 1.0f / sqrtf(total / (float)d + eps);
    if (mine)
        fin_store4(out + (size_t)t * d + i, make_float4(a.x * scale * wv.x, a.y * scale * wv.y, a.z * scale * wv.z, a.w * scale * wv.w));
}

template <typename TO>
static int launch_finish_cluster4(const float* partial, int splits, const float* bias, float* x, const float* w, TO* out,
                                  int n, int d, int slice, float eps, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    const int threads = (slice / 4 + 31) / 32 * 32;
    cfg.gridDim = dim3(n * FIN_CLUSTER); cfg.blockDim = dim3(threads); cfg.dynamicSmemBytes = 0; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = FIN_CLUSTER; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = xr_pdl_enabled() ? 2 : 1;
    cudaLaunchKernelEx(&cfg, k_finish_add_rmsnorm_cluster4<TO>, partial, splits, n, bias, x, w, out, d, slice, eps);
    return xr_launch_status();
}

template <typename TO>
static int launch_finish_cluster(const float* partial, int splits, const float* bias, float* x, const float* w, TO* out,
                                 int n, int d, int slice, float eps, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n * FIN_CLUSTER); cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = 0; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = FIN_CLUSTER; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = xr_pdl_enabled() ? 2 : 1;
    if (slice <= 256) cudaLaunchKernelEx(&cfg, k_finish_add_rmsnorm_cluster<TO, 1>, partial, splits, n, bias, x, w, out, d, slice, eps);
    else if (slice <= 512) cudaLaunchKernelEx(&cfg, k_finish_add_rmsnorm_cluster<TO, 2>, partial, splits, n, bias, x, w, out, d, slice, eps);
    else cudaLaunchKernelEx(&cfg, k_finish_add_rmsnorm_cluster<TO, 4>, partial, splits, n, bias, x, w, out, d, slice, eps);
    return xr_launch_status();
}

XR_EXPORT int xr_finish_add_rmsnorm(const float* partial, int splits, const float* bias, float* x, const float* w, void* out,
                                    int out_dtype, int n, int d, float eps, cudaStream_t stream) {
    if (n < 1 || d < 1 || splits < 1) return XR_ERR_ARG;
    if (out_dtype != XR_F32 && out_dtype != XR_BF16) return XR_ERR_ARG;
    const int slice = (d + FIN_CLUSTER - 1) / FIN_CLUSTER;
    const bool aligned = (((uintptr_t)partial | (uintptr_t)x | (uintptr_t)w | (uintptr_t)out | (uintptr_t)bias) & 15) == 0;
    if (n > 16 && n <= 64 && d >= 512 && (d % (4 * FIN_CLUSTER)) == 0 && d <= 4 * 256 * FIN_CLUSTER && aligned) {
        // 17 to 64 tokens: a cluster of eight blocks per token, each thread one quadruple of its block's slice (measured at
        // width 4096: 5.3 us against 8.4 us for the scalar cluster kernel at 64 tokens; up to 16 tokens the scalar kernel,
        // which is tuned for the latency of a single wave, is the faster one: 4.3 against 4.7 us at 8 tokens)
        if (out_dtype == XR_F32) return launch_finish_cluster4<float>(partial, splits, bias, x, w, (float*)out, n, d, d / FIN_CLUSTER, eps, stream);
        return launch_finish_cluster4<__nv_bfloat16>(partial, splits, bias, x, w, (__nv_bfloat16*)out, n, d, d / FIN_CLUSTER, eps, stream);
    }
    if (n > 64 && (d & 3) == 0 && d >= 1024 && d <= 4 * FIN_V4_PER * 1024 && aligned) {
        // many tokens: throughput counts, one block of (up to) 1024 threads per token, 16-byte vectors
        int threads = ((d / 4 + FIN_V4_PER - 1) / FIN_V4_PER + 31) / 32 * 32;
        if (threads > 1024) threads = 1024;
        if (out_dtype == XR_F32) xr_launch((k_finish_add_rmsnorm_vec4<float>), dim3(n), dim3(threads), 0, stream, partial, splits, n, bias, x, w, (float*)out, d, eps);
        else xr_launch((k_finish_add_rmsnorm_vec4<__nv_bfloat16>), dim3(n), dim3(threads), 0, stream, partial, splits, n, bias, x, w, (__nv_bfloat16*)out, d, eps);
        return xr_launch_status();
    }
    if (n <= 64 && d >= 512 && slice <= FIN_CL_PER * 256) {      // few tokens and a row worth cutting up
        if (out_dtype == XR_F32) return launch_finish_cluster<float>(partial, splits, bias, x, w, (float*)out, n, d, slice, eps, stream);
        return launch_finish_cluster<__nv_bfloat16>(partial, splits, bias, x, w, (__nv_bfloat16*)out, n, d, slice, eps, stream);
    }
    int threads = d >= 4096 ? 1024 : (d >= 1024 ? 512 : 256);      // few tokens, so many threads per token
    if (out_dtype == XR_F32) xr_launch((k_finish_add_rmsnorm<float>), dim3(n), dim3(threads), 0, stream, partial, splits, n, bias, x, w, (float*)out, d, eps);
    else xr_launch((k_finish_add_rmsnorm<__nv_bfloat16>), dim3(n), dim3(threads), 0, stream, partial, splits, n, bias, x, w, (__nv_bfloat16*)out, d, eps);
    return xr_launch_status();
}

// Plain finish for callers that need the sum itself: out (+)= sum of partials (+ bias).
template <typename TO, bool ACCUM>
__global__ void k_finish_plain(const float* __restrict__ partial, int splits, int n, int width, const float* __restrict__ bias,
                               TO* __restrict__ out, long long ldo) {
    xr_pdl_launch();
    xr_pdl_wait();
    size_t total = (size_t)n * width;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        size_t t = i / width, r = i % width;
        float v = 0.f;
        for (int s0 = 0; s0 < splits; s0 += 8) {
            float a[8];
#pragma unroll
            for (int q = 0; q < 8; q++) a[q] = xr_ld_now(partial + ((size_t)min(s0 + q, splits - 1) * n + t) * width + r);
#pragma unroll
            for (int q = 0; q < 8; q++) xr_ld_fence(a[q]);
#pragma unroll
            for (int q = 0; q < 8; q++) v += s0 + q < splits ? a[q] : 0.f;
        }
        if (bias) v += bias[r];
        size_t o = t * ldo + r;
        if (ACCUM) out[o] = xr_from_f32<TO>(xr_to_f32<TO>(out[o]) + v);
        else out[o] = xr_from_f32<TO>(v);
    }
}

XR_EXPORT int xr_finish_plain(const float* partial, int splits, const float* bias, void* out, int out_dtype, int accumulate,
                              int n, int width, long long ldo, cudaStream_t stream) {
    if (n < 1 || width < 1 || splits < 1 || ldo < width) return XR_ERR_ARG;
    size_t total = (size_t)n * width;
    int blocks = (int)((total + 255) / 256 < xr_sm_count() * 8 ? (total + 255) / 256 : xr_sm_count() * 8);
    if (accumulate) {
        if (out_dtype != XR_F32) return XR_ERR_ARG;
        xr_launch((k_finish_plain<float, true>), dim3(blocks), dim3(256), 0, stream, partial, splits, n, width, bias, (float*)out, ldo);
    } else if (out_dtype == XR_F32) {
        xr_launch((k_finish_plain<float, false>), dim3(blocks), dim3(256), 0, stream, partial, splits, n, width, bias, (float*)out, ldo);
    } else if (out_dtype == XR_BF16) {
        xr_launch((k_finish_plain<__nv_bfloat16, false>), dim3(blocks), dim3(256), 0, stream, partial, splits, n, width, bias, (__nv_bfloat16*)out, ldo);
    } else {
        return XR_ERR_ARG;
    }
    return xr_launch_status();
}

// QKV finish + rotation + page store.  One block per (token, head); head < H: query, < H + K: key, else value.
struct FinishRopeArgs {
    const float* partial; int splits; const float* bias;
    __nv_bfloat16* qkv;              // Q heads are written here (row stride (H + 2K) * hd); K and V too when cache_k is null
    const int* positions; const int* tok_seg; const int* block_tables; const float* inv_freq;
    __nv_bfloat16* cache_k; long long page_stride, v_offset;
    int n, H, K, hd, rotary_dim, max_pages, page_size;
    int adjacent;                    // pairs (2j, 2j + 1) instead of (j, j + rotary_dim/2)
    float mscale;                    // factor on the cosines and sines
};

__global__ void k_finish_rope_store(FinishRopeArgs a) {
    xr_pdl_launch();
    // The step's description (positions, block tables) and the rotation's frequencies do not change while the step
    // runs: where this token's rows go, and its angles, are worked out before the kernel ahead is complete.
    int t = blockIdx.x, head = blockIdx.y;
    int qkv_dim = (a.H + 2 * a.K) * a.hd;
    int col0 = head * a.hd;
    int pos = a.positions[t];
    int half = a.rotary_dim >> 1;
    bool is_q = head < a.H, is_k = !is_q && head < a.H + a.K;
    __nv_bfloat16* dst = a.qkv + (size_t)t * qkv_dim + col0;
    if (!is_q && a.cache_k != nullptr) {
        int kvh = is_k ? head - a.H : head - a.H - a.K;
        int page = a.block_tables[(size_t)a.tok_seg[t] * a.max_pages + pos / a.page_size];
        dst = a.cache_k + (size_t)page * a.page_stride + (is_k ? 0 : a.v_offset) + ((size_t)kvh * a.page_size + (pos % a.page_size)) * a.hd;
    }
    // A thread's unit is a pair (its index below half, in a head that is rotated) or a single element that is not
    // rotated (the tail of a Q or K head beyond the rotated width, and all of V).
    const bool rotated = is_q || is_k;
    const int j_mine = threadIdx.x;                            // the block is as wide as the head for the usual head sizes
    float cos_mine = 1.f, sin_mine = 0.f;
    if (j_mine < half && rotated) {
        float ang = (float)pos * a.inv_freq[j_mine];
        cos_mine = cosf(ang) * a.mscale; sin_mine = sinf(ang) * a.mscale;
    }
    xr_pdl_wait();
    const int units = rotated ? a.hd - half : a.hd;            // pairs first, then the elements beyond them
    for (int u = threadIdx.x; u < units; u += blockDim.x) {
        const bool pair = rotated && u < half;
        const int i0 = pair ? (a.adjacent ? 2 * u : u) : (rotated ? u + half : u);
        const int i1 = pair ? (a.adjacent ? 2 * u + 1 : u + half) : i0;
        // the loads of eight splits are in flight together (indices clamped, so that none is conditional); the sums
        // are taken in split order
        float v0 = 0.f, v1 = 0.f;
        const size_t split_stride = (size_t)a.n * qkv_dim;
        const float* p0 = a.partial + (size_t)t * qkv_dim + col0;
        for (int s0 = 0; s0 < a.splits; s0 += 8) {
            float x0[8], x1[8];
#pragma unroll
            for (int q = 0; q < 8; q++) {
                const float* p = p0 + (size_t)min(s0 + q, a.splits - 1) * split_stride;
                x0[q] = xr_ld_now(p + i0);
                x1[q] = xr_ld_now(p + i1);
            }
#pragma unroll
            for (int q = 0; q < 8; q++) { xr_ld_fence(x0[q]); xr_ld_fence(x1[q]); }
#pragma unroll
            for (int q = 0; q < 8; q++) {
                const bool live = s0 + q < a.splits;
                v0 += live ? x0[q] : 0.f;
                v1 += (live && pair) ? x1[q] : 0.f;
            }
        }
        if (a.bias) { v0 += a.bias[col0 + i0]; if (pair) v1 += a.bias[col0 + i1]; }
        if (pair) {
            // the product's output is rounded to the activation dtype before the rotation, as on the unfused path
            v0 = __bfloat162float(__float2bfloat16_rn(v0)); v1 = __bfloat162float(__float2bfloat16_rn(v1));
            float c = cos_mine, s = sin_mine;
            if (u != j_mine) {                                // a head wider than the block: later rounds
                float ang = (float)pos * a.inv_freq[u];
                c = cosf(ang) * a.mscale; s = sinf(ang) * a.mscale;
            }
            dst[i0] = __float2bfloat16_rn(v0 * c - v1 * s);
            dst[i1] = __float2bfloat16_rn(v0 * s + v1 * c);
        } else {
            dst[i0] = __float2bfloat16_rn(v0);
        }
    }
}

// The same for steps of more than 16 tokens, where one block per (token, head) means thousands of small blocks that keep
// the kernel after this one off the machine.  A thread takes four neighbouring pairs (j .. j + 3 with j + half ..) or
// four neighbouring elements that are not rotated, with the 16-byte loads of up to eight splits in flight together; a
// block takes 256 such units of one token.  Pairs (j, j + half) only; sums, roundings and products as above, in the same order.
__global__ void __launch_bounds__(256) k_finish_rope_store_vec4(FinishRopeArgs a) {
    xr_pdl_launch();
    const int t = blockIdx.x;
    const int half = a.rotary_dim >> 1, pair_units = half >> 2;
    const int uq = (a.hd - half) >> 2, uv = a.hd >> 2;             // units of a rotated head and of a value head
    const int rot_heads = a.H + a.K;
    const int g = blockIdx.y * 256 + threadIdx.x;
    if (g >= rot_heads * uq + a.K * uv) return;
    int head, u;
    const bool rotated = g < rot_heads * uq;
    if (rotated) { head = g / uq; u = g - head * uq; }
    else { const int r = g - rot_heads * uq; head = rot_heads + r / uv; u = r % uv; }
    const bool pair = rotated && u < pair_units;
    const int i0 = pair ? 4 * u : (rotated ? 2 * half + 4 * (u - pair_units) : 4 * u);
    const int i1 = i0 + half;
    const int qkv_dim = (a.H + 2 * a.K) * a.hd, col0 = head * a.hd;
    const int pos = a.positions[t];
    __nv_bfloat16* dst = a.qkv + (size_t)t * qkv_dim + col0;
    if (head >= a.H && a.cache_k != nullptr) {
        const bool is_k = head < rot_heads;
        const int kvh = is_k ? head - a.H : head - rot_heads;
        const int page = a.block_tables[(size_t)a.tok_seg[t] * a.max_pages + pos / a.page_size];
        dst = a.cache_k + (size_t)page * a.page_stride + (is_k ? 0 : a.v_offset) + ((size_t)kvh * a.page_size + (pos % a.page_size)) * a.hd;
    }
    float c[4] = {1.f, 1.f, 1.f, 1.f}, sn[4] = {0.f, 0.f, 0.f, 0.f};
    if (pair) {
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const float ang = (float)pos * a.inv_freq[i0 + e];
            c[e] = cosf(ang) * a.mscale; sn[e] = sinf(ang) * a.mscale;
        }
    }
    xr_pdl_wait();
    float4 v0 = make_float4(0.f, 0.f, 0.f, 0.f), v1 = v0;
    const size_t split_stride = (size_t)a.n * qkv_dim;
    const float* p0 = a.partial + (size_t)t * qkv_dim + col0;
    for (int s0 = 0; s0 < a.splits; s0 += 8) {
        float4 x0[8], x1[8];
#pragma unroll
        for (int q = 0; q < 8; q++) {
            const float* p = p0 + (size_t)min(s0 + q, a.splits - 1) * split_stride;
            x0[q] = xr_ld_now4(reinterpret_cast<const float4*>(p + i0));
            x1[q] = xr_ld_now4(reinterpret_cast<const float4*>(p + (pair ? i1 : i0)));
        }
#pragma unroll
        for (int q = 0; q < 8; q++) { xr_ld_fence(x0[q]); xr_ld_fence(x1[q]); }
#pragma unroll
        for (int q = 0; q < 8; q++) {
            if (s0 + q < a.splits) {
                v0.x += x0[q].x; v0.y += x0[q].y; v0.z += x0[q].z; v0.w += x0[q].w;
                if (pair) { v1.x += x1[q].x; v1.y += x1[q].y; v1.z += x1[q].z; v1.w += x1[q].w; }
            }
        }
    }
    float a0[4] = {v0.x, v0.y, v0.z, v0.w}, a1[4] = {v1.x, v1.y, v1.z, v1.w};
    if (a.bias) {
#pragma unroll
        for (int e = 0; e < 4; e++) { a0[e] += a.bias[col0 + i0 + e]; if (pair) a1[e] += a.bias[col0 + i1 + e]; }
    }
    __nv_bfloat16 o0[4], o1[4];
#pragma unroll
    for (int e = 0; e < 4; e++) {
        if (pair) {
            // the product's output is rounded to the activation dtype before the rotation, as on the unfused path
            const float r0 = __bfloat162float(__float2bfloat16_rn(a0[e])), r1 = __bfloat162float(__float2bfloat16_rn(a1[e]));
            o0[e] = __float2bfloat16_rn(r0 * c[e] - r1 * sn[e]);
            o1[e] = __float2bfloat16_rn(r0 * sn[e] + r1 * c[e]);
        } else {
            o0[e] = __float2bfloat16_rn(a0[e]);
        }
    }
    *reinterpret_cast<uint2*>(dst + i0) = *reinterpret_cast<const uint2*>(o0);
    if (pair) *reinterpret_cast<uint2*>(dst + i1) = *reinterpret_cast<const uint2*>(o1);
}

XR_EXPORT int xr_finish_rope_store(const float* partial, int splits, const float* bias, void* qkv, const int* positions,
                                   const int* tok_seg, const int* block_tables, const float* inv_freq, void* cache_k,
                                   long long page_stride, long long v_offset, int n, int H, int K, int hd, int rotary_dim,
                                   int max_pages, int page_size, int adjacent_pairs, float mscale, cudaStream_t stream) {
    if (n < 1 || H < 1 || K < 1 || hd < 1 || rotary_dim < 0 || rotary_dim > hd || (rotary_dim & 1) || page_size < 1 ||
        splits < 1 || H + 2 * K > 65535)
        return XR_ERR_ARG;
    FinishRopeArgs a{partial, splits, bias, (__nv_bfloat16*)qkv, positions, tok_seg, block_tables, inv_freq,
                     (__nv_bfloat16*)cache_k, page_stride, v_offset, n, H, K, hd, rotary_dim, max_pages, page_size,
                     adjacent_pairs ? 1 : 0, mscale};
    const int half = rotary_dim >> 1;
    if (n > 16 && !adjacent_pairs && hd % 4 == 0 && half % 4 == 0 && ((uintptr_t)partial & 15) == 0 && ((uintptr_t)qkv & 7) == 0 &&
        ((uintptr_t)cache_k & 7) == 0 && page_stride % 4 == 0 && v_offset % 4 == 0) {
        const int units = (H + K) * ((hd - half) >> 2) + K * (hd >> 2);
        xr_launch(k_finish_rope_store_vec4, dim3(n, (units + 255) / 256), dim3(256), 0, stream, a);
        return xr_launch_status();
    }
    int threads = hd >= 128 ? 128 : (hd >= 64 ? 64 : 32);
    xr_launch(k_finish_rope_store, dim3(n, H + 2 * K), dim3(threads), 0, stream, a);
    return xr_launch_status();
}
