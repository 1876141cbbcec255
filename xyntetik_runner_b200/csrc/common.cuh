// Shared helpers of the sm_100a kernels: dtype codes, conversions, reductions.
//
// Every launcher is `extern "C"`, takes raw device pointers, explicit extents
// and a stream, and returns 0 or a negative error code (see XR_ERR_*); the
// Python side turns a non-zero code into an exception.  No launcher
// allocates.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define XR_F32 0
#define XR_BF16 1

#define XR_OK 0
#define XR_ERR_ARG (-1)        // a size or dtype the kernel refuses
#define XR_ERR_LAUNCH (-2)     // the runtime refused the launch (cudaGetLastError)

#define XR_EXPORT extern "C" __attribute__((visibility("default")))

// Programmatic dependent launch: a kernel launched through xr_launch may be scheduled while the kernel before
// it in the stream is still in its last wave; it must call xr_pdl_wait() before it touches global memory
// (the wait returns when the earlier kernel has completed and its writes are visible) and calls
// xr_pdl_launch() to let the kernel after it start the same way.  Launch latency and block scheduling of
// back-to-back kernels then overlap instead of adding up.  XRB200_NO_PDL=1 turns the attribute off.
#ifndef XR_TRACE
__device__ __forceinline__ void xr_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#else
// Tracing build (see build.py): thread 0 of block 0 of every launch records the time it reached the wait (it
// was resident then), the time the wait returned (the kernel ahead was complete) and the launch's shape.  Each
// source file has its own record; xr_trace_dump (elementwise.cu) collects them through the functions registered here.
static __device__ unsigned long long xr_tr_buf[4096 * 4];
static __device__ unsigned int xr_tr_n;
typedef int (*xr_tr_dump_fn)(unsigned long long*, unsigned int*);
extern "C" int xr_trace_add(xr_tr_dump_fn fn);
static int xr_tr_dump_local(unsigned long long* host, unsigned int* n) {
    cudaMemcpyFromSymbol(n, xr_tr_n, sizeof(unsigned int));
    cudaMemcpyFromSymbol(host, xr_tr_buf, sizeof(xr_tr_buf));
    unsigned int zero = 0;
    cudaMemcpyToSymbol(xr_tr_n, &zero, sizeof(unsigned int));
    return 0;
}
static int xr_tr_registered = xr_trace_add(xr_tr_dump_local);
__device__ __forceinline__ void xr_pdl_wait() {
    const bool me = (blockIdx.x | blockIdx.y | blockIdx.z) == 0 && threadIdx.x == 0;
    unsigned long long t0 = 0, t1 = 0;
    if (me) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (me) {
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        unsigned int i = atomicAdd(&xr_tr_n, 1u);
        if (i < 4096) {
            xr_tr_buf[4 * i] = t0; xr_tr_buf[4 * i + 1] = t1;
            xr_tr_buf[4 * i + 2] = ((unsigned long long)gridDim.x << 40) | ((unsigned long long)gridDim.y << 20) | gridDim.z;
            xr_tr_buf[4 * i + 3] = blockDim.x;
        }
    }
}
#endif
__device__ __forceinline__ void xr_pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#include <stdlib.h>
#include <stdio.h>
static inline bool xr_pdl_enabled() {
    static int on = -1;
    if (on < 0) { const char* e = getenv("XRB200_NO_PDL"); on = (e && e[0] && e[0] != '0') ? 0 : 1; }
    return on == 1;
}

// Streaming multiprocessors of the current device (asked once per device): grids and wave models are sized by
// it, so a part exposed with fewer of them than the full chip is not over-subscribed.
static inline int xr_sm_count() {
    static int known[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (known[dev] == 0) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v < 1) v = 148;
        known[dev] = v;
    }
    return known[dev];
}

// Tensor maps (TMA descriptors) that were encoded before.  A step encodes the same few dozen maps again and again (the
// weights of each layer, the buffers that keep their addresses, the cache groups), and an encode costs the host a
// few microseconds each, which a step of a few hundred tokens does not hide.  The key is everything the encode is
// given; a slot is taken by its key's hash and simply overwritten by another key that lands there.  `Map` is
// CUtensorMap (this header does not include cuda.h); `encode(&map)` makes the map and says whether it could.
struct XrMapKey {
    const void* base;
    unsigned long long dims[3], strides[2];
    unsigned box[3], rank, flavour;
    bool operator==(const XrMapKey& o) const {
        return base == o.base && dims[0] == o.dims[0] && dims[1] == o.dims[1] && dims[2] == o.dims[2] && strides[0] == o.strides[0] &&
               strides[1] == o.strides[1] && box[0] == o.box[0] && box[1] == o.box[1] && box[2] == o.box[2] && rank == o.rank && flavour == o.flavour;
    }
};
template <typename Map, typename Encode>
static inline bool xr_cached_map(Map* out, const XrMapKey& key, Encode encode) {
    constexpr int SLOTS = 1024;
    struct Slot { XrMapKey key; Map map; bool full; };
    static Slot* slots = nullptr;                 // (one table per kind of map and source file; never freed)
    static volatile int busy = 0;
    unsigned long long h = (unsigned long long)(uintptr_t)key.base * 0x9E3779B97F4A7C15ull;
    h ^= (key.dims[0] * 31 + key.dims[1]) * 0xC2B2AE3D27D4EB4Full + key.strides[0] * 0x165667B19E3779F9ull + key.box[1] * 131 + key.flavour;
    const int at = (int)((h >> 32) % SLOTS);
    while (__sync_lock_test_and_set(&busy, 1)) {}           // calls from two host threads are rare and short
    if (!slots) slots = new Slot[SLOTS]();
    bool ok = true;
    if (slots[at].full && slots[at].key == key) {
        *out = slots[at].map;
    } else {
        ok = encode(out);
        if (ok) { slots[at].key = key; slots[at].map = *out; slots[at].full = true; }
    }
    __sync_lock_release(&busy);
    return ok;
}

template <typename... KArgs, typename... Args>
static inline void xr_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = xr_pdl_enabled() ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

static inline int xr_launch_status() {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) fprintf(stderr, "[xrb200] the runtime refused a launch: %s\n", cudaGetErrorString(e));
    return e == cudaSuccess ? XR_OK : XR_ERR_LAUNCH;
}

// Loads that stay where they are written.  Left to itself the compiler interleaves a run of independent loads with
// the arithmetic that consumes them (it saves registers), and a latency-bound kernel then pays one trip to L2 per
// load instead of one per run.  A run of xr_ld_now() calls is issued back to back; xr_ld_fence() on each value
// after the run keeps every later use behind all of the loads.
__device__ __forceinline__ float xr_ld_now(const float* p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float4 xr_ld_now4(const float4* p) {
    float4 v;
    asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void xr_ld_fence(float& v) { asm volatile("" : "+f"(v)); }
__device__ __forceinline__ void xr_ld_fence(float4& v) { asm volatile("" : "+f"(v.x), "+f"(v.y), "+f"(v.z), "+f"(v.w)); }

template <typename T> __device__ __forceinline__ float xr_to_f32(T v);
template <> __device__ __forceinline__ float xr_to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float xr_to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T xr_from_f32(float v);
template <> __device__ __forceinline__ float xr_from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 xr_from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float xr_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float xr_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The
// order of additions depends only on the block size, never on the data.
__device__ __forceinline__ float xr_block_sum(float v, float* scratch /* >= 33 floats */) {
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = xr_warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? scratch[lane] : 0.f;
        t = xr_warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}
