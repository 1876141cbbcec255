// out[t][r] = sum_k X[t][k] * W[r][k] on the 5th-generation tensor cores (tcgen05), bfloat16 in,
// float32 accumulation in tensor memory.
//
// The weight matrix is the M operand: a CTA owns 128 rows of W (output features) and BN tokens
// (BN = 16..256, the N of the instruction), so the same kernel serves a decode step of one token
// (weights stream through once, tokens are padding-free up to 16) and a 2,048-token prefill
// (128 x 256 tiles).  Both operands are K-major in global memory, which is what TMA with the
// 128-byte swizzle and the K-major shared-memory descriptor want: no transposes anywhere.
//
// Roles inside a CTA of 320 threads (192 for the 16-token tile, 576 in the CTA-pair kernel):
//   warp 0, one lane : TMA producer  (cp.async.bulk.tensor.2d -> shared, completes on an mbarrier)
//   warp 1, one lane : MMA issuer    (tcgen05.mma, commits free the stage / signal the epilogue);
//                      the warp also allocates and frees tensor memory
//   warps 2..        : epilogue      (tcgen05.ld of their 32 lanes, then global stores); a warp may only
//                      read the 32 tensor-memory lanes of its index mod 4, so the warps of a quarter
//                      take alternate 16-column chunks
// A K loop over 64-element blocks runs through a ring of shared-memory stages.  Steps of more than 128 tokens
// run on pairs of CTAs (k_gemm_tc_pair below): persistent clusters of two, one instruction across both.
//
// Epilogues: store (bfloat16 or float32, optional bias, optional activation), add into the float32 residual
// stream, gated (h = act(g) * u: the packed matrix interleaves gate and up rows so that one 128-row tile holds
// 64 features, sixteen gate rows beside their sixteen up rows in every quarter of the accumulator's lanes; a
// thread gets its partner's half by warp shuffles and the [n, 2F] intermediate never exists), or a split-K
// partial to scratch that `k_splitk_finish` sums in a fixed order and finishes with the same epilogues.
// Activations: none, SiLU (0 below -80, src/model.c:4451-4452), tanh-GELU (src/model.c:4438-4441).
//
// Every wait on an mbarrier is bounded: after XR_SPIN_LIMIT polls the waiter raises the CTA's abort
// flag, every role leaves its loop, in-flight copies are waited for (bounded again), tensor memory is
// freed, and the kernel records the failure in a status word that the launcher's caller reads.
//
// The reference multiplies bf16 weights with scalar FMA kernels (`k_mv_bf16`, `k_mv_bf16_b`,
// src/kernels.cu:534-549; `k_gemvb_bf16_x4/_x8`, src/kernels.cu:2814-2852) and adds the residual and
// the activation in kernels of their own (`k_add` :2903, `k_silu_mul` :2868).
#include "common.cuh"
#include <cuda.h>

#define TC_BM 128          // W rows per CTA (the M of the instruction)
#define TC_BK 64           // K elements per stage: 128 bytes, one swizzle atom
#define TC_THREADS 320       // producer warp, MMA warp, eight epilogue warps
// a tile of 16 tokens is one chunk of accumulator columns: four epilogue warps are all it can use
__host__ __device__ constexpr int tc_threads(int bn) { return bn <= 16 ? 192 : TC_THREADS; }
#define XR_SPIN_LIMIT (1u << 24)

#define TC_EPI_STORE 0     // out[t][r] = acc (+ bias), bfloat16 or float32
#define TC_EPI_ADD 1       // out[t][r] += acc (+ bias), float32 residual stream
#define TC_EPI_GATED 2     // out[t][f] = act(acc of gate row f) * (acc of up row f); W packed with the rows interleaved
#define TC_EPI_PARTIAL 3   // scratch[split][t][r] = acc (float32), r a row of the product as it is packed

#define TC_ACT_NONE 0
#define TC_ACT_SILU 1
#define TC_ACT_GELU_TANH 2

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when it gave up (or another role already had).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < XR_SPIN_LIMIT; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, float* v) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]);
}

// silu(g) = g / (1 + exp(-g)), 0 below -80 (src/model.c:4451-4452), with the hardware's approximate exp2 and
// reciprocal: their error (about 2^-22) disappears in the bfloat16 rounding of the result, and an epilogue that
// spends hundreds of instructions per element on exact exp and division holds the tensor core up.
__device__ __forceinline__ float tc_silu(float g) {
    return g < -80.0f ? 0.0f : __fdividef(g, 1.0f + __expf(-g));
}
// tanh-GELU: 0.5 g (1 + tanh(0.7978845608 (g + 0.044715 g^3))) (src/model.c:4438-4441), tanh by the hardware's
// approximation for the same reason
__device__ __forceinline__ float tc_gelu_tanh(float g) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.7978845608f * (g + 0.044715f * g * g * g)));
    return 0.5f * g * (1.0f + t);
}
__device__ __forceinline__ float tc_act(int act, float g) {
    return act == TC_ACT_SILU ? tc_silu(g) : (act == TC_ACT_GELU_TANH ? tc_gelu_tanh(g) : g);
}

// K-major operand tile in shared memory, rows of 128 bytes, 128-byte swizzle, groups of 8 rows 1024 bytes
// apart: start address and offsets in 16-byte units, descriptor version 1 (bit 46), layout type 2 (bits 61-63).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;                 // leading byte offset (unused with a swizzled K-major tile)
    d |= (uint64_t)(1024 >> 4) << 32;       // stride byte offset: 8 rows
    d |= (uint64_t)1 << 46;                 // descriptor version
    d |= (uint64_t)2 << 61;                 // SWIZZLE_128B
    return d;
}
// kind::f16 instruction descriptor: D float32, A and B bfloat16, both K-major, M = 128, N = bn.
__host__ __device__ constexpr uint32_t instr_desc(int bn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
}

struct TcParams {
    void* out;                  // see TC_EPI_*
    const float* bias;          // [n_out] or null
    float* partial;             // split-K scratch
    int* status;                // device word: non-zero when a wait gave up
    long long ldo;              // row stride of out in elements
    int n, n_out, K;            // tokens, output features (gated: features, the product has 128 rows per 64 of them), reduction length
    int splits;                 // z-slices of the grid; slice z handles K blocks [z*total/splits, (z+1)*total/splits)
    int epilogue, out_dtype;
    int act;                    // TC_ACT_*: applied to the stored value (store epilogue) or to the gate (gated epilogue)
    int gated;                  // the product's rows are gate and up rows interleaved (also when the epilogue is PARTIAL)
    int bn;                     // tokens per tile: a multiple of 16, at most the kernel's BN (which sizes the buffers)
    int packed;                 // W is stored tile by tile: [row tile][K block][128][64], see xr_gemm_tc
    int w_kblocks;              // packed: K blocks per row tile in the packed array
    int tok_tiles, pair_tiles;  // CTA-pair kernel: token tiles, and tiles in all (token tiles x pairs of row tiles)
};

// ---------------------------------------------------------------------------------------------
// Epilogue of one tile, run by warps 2..9 once the accumulator is complete.  A warp may only read the 32
// tensor-memory lanes of its index mod 4, so two warps share each quarter and take alternate 16-column
// chunks (with sixteen epilogue warps, four share a quarter).
//
// Gated products: quarter q of the tile's 128 rows holds the gate rows of features 64 tile + 16 q + (0..15) in its
// lanes 0..15 and their up rows in lanes 16..31.  Of a 16-column chunk the gate lanes finish columns 0..7 and the
// up lanes columns 8..15; each gets the other half of what it needs from its partner lane (lane xor 16) by shuffle.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tc_epilogue(const TcParams& p, uint32_t tmem_base, int row0, int tok0, int warp, int lane,
                                            int warps_per_quarter = 2, int split = (int)blockIdx.z) {
    const int quad = warp & 3, chunk_first = (warp - 2) >> 2;
    const int r = row0 + quad * 32 + lane;            // row of the product that this thread's lane holds
    const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16);
    const bool gated_out = p.epilogue == TC_EPI_GATED;
    // feature of a gated product: 64 per 128-row tile, 16 per quarter
    const int f = (row0 >> 1) + quad * 16 + (lane & 15), up_lane = lane >> 4;
    const bool row_ok = gated_out ? f < p.n_out : r < (p.gated ? ((p.n_out + 63) / 64) * 128 : p.n_out);
    const float b = (p.bias != nullptr && row_ok && (p.epilogue == TC_EPI_STORE || p.epilogue == TC_EPI_ADD) && split == 0)
                        ? p.bias[r] : 0.f;
#pragma unroll 1
    for (int c0 = chunk_first * 16; c0 < p.bn; c0 += 16 * warps_per_quarter) {
        if (tok0 + c0 >= p.n) break;               // warp-uniform
        float g[16];
        tc_ld16(taddr + c0, g);
        if (gated_out) {
            // gate lanes send their columns 8..15 and receive the up values of columns 0..7; up lanes the reverse
            float other[8];
#pragma unroll
            for (int c = 0; c < 8; c++) other[c] = __shfl_xor_sync(0xffffffffu, up_lane ? g[c] : g[8 + c], 16);
            if (!row_ok) continue;
            const int col0 = tok0 + c0 + (up_lane ? 8 : 0);
            float v[8];
#pragma unroll
            for (int c = 0; c < 8; c++) v[c] = up_lane ? tc_act(p.act, other[c]) * g[8 + c] : tc_act(p.act, g[c]) * other[c];
            if (p.out_dtype == XR_BF16) {
                __nv_bfloat16* dst = (__nv_bfloat16*)p.out + (size_t)col0 * p.ldo + f;
#pragma unroll
                for (int c = 0; c < 8; c++)
                    if (col0 + c < p.n) dst[(size_t)c * p.ldo] = __float2bfloat16_rn(v[c]);
            } else {
                float* dst = (float*)p.out + (size_t)col0 * p.ldo + f;
#pragma unroll
                for (int c = 0; c < 8; c++)
                    if (col0 + c < p.n) dst[(size_t)c * p.ldo] = v[c];
            }
            continue;
        }
        if (!row_ok) continue;
        if (p.epilogue == TC_EPI_ADD) {
            // read-modify-write of the float32 residual: all loads first, so that they overlap
            float* dst = (float*)p.out + (size_t)(tok0 + c0) * p.ldo + r;
            float old[16];
#pragma unroll
            for (int c = 0; c < 16; c++) old[c] = xr_ld_now(dst + (size_t)(tok0 + c0 + c < p.n ? c : 0) * p.ldo);
#pragma unroll
            for (int c = 0; c < 16; c++) xr_ld_fence(old[c]);
#pragma unroll
            for (int c = 0; c < 16; c++)
                if (tok0 + c0 + c < p.n) dst[(size_t)c * p.ldo] = old[c] + (g[c] + b);
            continue;
        }
        // a chunk that runs past the last token stores only what exists
        const int live = p.n - (tok0 + c0) < 16 ? p.n - (tok0 + c0) : 16;
        if (p.epilogue == TC_EPI_PARTIAL) {
            const size_t width = p.gated ? (size_t)((p.n_out + 63) / 64) * 128 : (size_t)p.n_out;
            float* dst = p.partial + ((size_t)split * p.n + tok0 + c0) * width + r;
#pragma unroll
            for (int c = 0; c < 16; c++)
                if (c < live) dst[(size_t)c * width] = g[c];
            continue;
        }
        float v[16];
#pragma unroll
        for (int c = 0; c < 16; c++) v[c] = tc_act(p.act, g[c] + b);
        if (p.out_dtype == XR_BF16) {
            __nv_bfloat16* dst = (__nv_bfloat16*)p.out + (size_t)(tok0 + c0) * p.ldo + r;
#pragma unroll
            for (int c = 0; c < 16; c++)
                if (c < live) dst[(size_t)c * p.ldo] = __float2bfloat16_rn(v[c]);
        } else {
            float* dst = (float*)p.out + (size_t)(tok0 + c0) * p.ldo + r;
#pragma unroll
            for (int c = 0; c < 16; c++)
                if (c < live) dst[(size_t)c * p.ldo] = v[c];
        }
    }
}

// ---------------------------------------------------------------------------------------------
// The kernel.  grid = (token tiles, row tiles, K splits): the CTAs that share a tile of W are neighbours in
// launch order, so W comes from HBM once and from L2 for the others.
// ---------------------------------------------------------------------------------------------
template <int BN, int STAGES, int MINB>
__global__ void __launch_bounds__(tc_threads(BN), MINB)
k_gemm_tc(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, TcParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    constexpr int W_BYTES = TC_BM * TC_BK * 2;
    constexpr int X_BYTES = BN * TC_BK * 2;
    constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
    constexpr int ACC_COLS = BN;
    constexpr int TMEM_COLS = ACC_COLS <= 32 ? 32 : (ACC_COLS <= 64 ? 64 : (ACC_COLS <= 128 ? 128 : (ACC_COLS <= 256 ? 256 : 512)));
    // carve shared memory: stages (1024-byte aligned), then barriers
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(smem + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_ready = empty + STAGES;
    uint32_t* tmem_slot = (uint32_t*)(acc_ready + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.y * TC_BM, tok0 = blockIdx.x * p.bn;
    const int total_kb = (p.K + TC_BK - 1) / TC_BK;
    const int kb0 = (int)(((long long)blockIdx.z * total_kb) / p.splits);
    const int kb1 = (int)(((long long)(blockIdx.z + 1) * total_kb) / p.splits);
    const int nkb = kb1 - kb0;                     // >= 1: splits <= total_kb

    xr_pdl_launch();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(acc_ready, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Everything above touched no global memory.  The weights are constants, so the producer fills its ring with
    // them before the kernel ahead in the stream is known to be complete; the tokens are read only after that.
    auto load_w = [&](int i) {
        int s = i % STAGES;
        uint8_t* st = smem + s * STAGE_BYTES;
        mbar_expect_tx(&full[s], W_BYTES + p.bn * TC_BK * 2);
        if (p.packed) {
            // tile (row tile, K block) is 128 consecutive rows of 64 elements: one contiguous 16 KB read
            tma_load_2d(st, &map_w, 0, (blockIdx.y * p.w_kblocks + kb0 + i) * TC_BM, &full[s]);
        } else {
            tma_load_2d(st, &map_w, (kb0 + i) * TC_BK, row0, &full[s]);
        }
    };
    const int early = nkb < STAGES ? nkb : STAGES;
    if (warp == 0 && lane == 0)
        for (int i = 0; i < early; i++) load_w(i);
    xr_pdl_wait();

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int issued = early;
            for (int i = 0; i < nkb; i++) {
                int s = i % STAGES;
                if (i >= STAGES) {
                    if (!mbar_wait(&empty[s], ((i / STAGES) - 1) & 1, abort_flag)) break;
                    load_w(i);
                }
                tma_load_2d(smem + s * STAGE_BYTES + W_BYTES, &map_x, (kb0 + i) * TC_BK, tok0, &full[s]);
                issued = i + 1;
            }
            if (*abort_flag) {
                // copies already issued still write shared memory: wait for them (bounded) before the CTA may exit
                for (int i = max(0, issued - STAGES); i < issued; i++)
                    for (uint32_t w = 0; w < XR_SPIN_LIMIT && !mbar_try_wait(&full[i % STAGES], (i / STAGES) & 1); w++) {}
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = instr_desc(p.bn);
            bool ok = true;
            for (int i = 0; i < nkb && ok; i++) {
                int s = i % STAGES;
                ok = mbar_wait(&full[s], (i / STAGES) & 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
                uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
                uint32_t b_addr = a_addr + W_BYTES;
#pragma unroll
                for (int k = 0; k < TC_BK / 16; k++)
                    tc_mma(tmem_base, smem_desc_sw128(a_addr + k * 32), smem_desc_sw128(b_addr + k * 32), idesc, (i > 0 || k > 0) ? 1u : 0u);
                tc_commit(&empty[s]);          // the stage is free once these MMAs have read it
            }
            if (ok) tc_commit(acc_ready);      // accumulators complete
        }
    } else {
        // ---------------- epilogue: warps 2..9 ----------------
        bool ok = mbar_wait(acc_ready, 0, abort_flag);
        tc_fence_after();
        if (ok) tc_epilogue(p, tmem_base, row0, tok0, warp, lane);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, 1);
}

// ---------------------------------------------------------------------------------------------
// The same product on pairs of CTAs (cta_group::2), for steps of many tokens.  A cluster of two CTAs owns
// 256 rows of W (128 each) and a tile of up to 256 tokens; each CTA stages its own rows of W and HALF of the
// tokens, and one instruction issued by the even CTA multiplies across both CTAs' shared memory into both
// CTAs' tensor memory (each gets its 128 rows x all tokens).  A CTA thus fetches 32 KB per K block instead of
// 48 KB for the same 128 x 256 outputs: the single-CTA kernel is bound by exactly that operand traffic.
//
// Barriers: the copies of both CTAs complete on the even CTA's `full` barrier (its producer announces the bytes
// of both); the even CTA's MMA warp releases a stage, and at the end the accumulators, with commits that arrive
// on the barrier of the same name in both CTAs.  Both CTAs allocate and free tensor memory together; a cluster
// barrier after set-up keeps a copy from completing on a barrier that is not initialised yet, and one before
// the end keeps a CTA from leaving while its partner may still signal it.  grid = 2 x clusters, cluster
// (2, 1, 1); a tile is (token tile, pair of row tiles), CTA `rank` of the pair owns row tile 2 x pair + rank.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t tc_cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void tc_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t tc_map_to_rank(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
// copy into this CTA's shared memory, completion counted on a barrier that may be the partner's
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {       // arrives on `bar` of both CTAs
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// M = 256 across the pair, N = bn
__host__ __device__ constexpr uint32_t instr_desc_pair(int bn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

#define TC2_BN 256         // token capacity of a pair's tile; each CTA stages half
#define TC2_THREADS 576    // producer warp, MMA warp, sixteen epilogue warps (the tile is wide: four per quarter)
__device__ __forceinline__ void mbar_arrive_remote(uint32_t bar_cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

// The pairs are persistent: `gridDim.x / 2` clusters (as many as the machine holds at once) walk the work items
// round-robin.  An item is a tile, or with `splits` > 1 one slice along K of a tile (steps of a few hundred tokens
// have fewer tiles than the machine has CTA pairs); items are ordered slice by slice and within a slice token tile
// fastest, so that clusters working at the same time share rows of W, and K ranges, in L2.  The ring
// of stages runs on across tiles (the producer fetches the next tile's operands while the epilogue of this one
// runs), and two accumulators are kept in tensor memory, so that the MMAs of the next tile overlap the epilogue
// too (a gated product as well: its gate and up rows are interleaved in one tile, so it has one accumulator a tile).
template <int STAGES>
__global__ void __launch_bounds__(TC2_THREADS, 1)
k_gemm_tc_pair(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, TcParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    constexpr int W_BYTES = TC_BM * TC_BK * 2;
    constexpr int X_BYTES = (TC2_BN / 2) * TC_BK * 2;
    constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
    constexpr int TMEM_COLS = 512;
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(smem + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;          // [2]
    uint64_t* acc_empty = acc_full + 2;           // [2], used in the even CTA only
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    xr_pdl_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = tc_cluster_rank();                 // 0: issues the MMAs
    const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
    const int half = p.bn >> 1;                              // tokens this CTA stages
    const int nkb = (p.K + TC_BK - 1) / TC_BK;
    const uint32_t stage_bytes = W_BYTES + half * TC_BK * 2;
    constexpr int ACC_BUFS = 2;                              // two accumulators of TC2_BN columns each

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; b++) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 2 * 16); }   // 16 epilogue warps x 2 CTAs
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    tc_cluster_sync();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    xr_pdl_wait();

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        if (lane == 0) {
            int it = 0;                                      // K blocks fetched so far, over all tiles
            bool ok = true;
            for (int item = cluster_id; item < p.pair_tiles * p.splits && ok; item += n_clusters) {
                const int tile = item % p.pair_tiles, split = item / p.pair_tiles;
                const int row_tile = 2 * (tile / p.tok_tiles) + (int)rank;
                const int tok0 = (tile % p.tok_tiles) * p.bn;
                const int kb0 = (int)(((long long)split * nkb) / p.splits), kb1 = (int)(((long long)(split + 1) * nkb) / p.splits);
                for (int i = kb0; i < kb1; i++, it++) {
                    int s = it % STAGES;
                    if (it >= STAGES && !mbar_wait(&empty[s], ((it / STAGES) - 1) & 1, abort_flag)) { ok = false; break; }
                    uint8_t* st = smem + s * STAGE_BYTES;
                    const uint32_t bar = tc_map_to_rank(smem_u32(&full[s]), 0);
                    if (rank == 0) mbar_expect_tx(&full[s], 2 * stage_bytes);
                    int kx = i * TC_BK;
                    if (p.packed) tma_load_2d_pair(st, &map_w, 0, (row_tile * p.w_kblocks + i) * TC_BM, bar);
                    else tma_load_2d_pair(st, &map_w, kx, row_tile * TC_BM, bar);
                    tma_load_2d_pair(st + W_BYTES, &map_x, kx, tok0 + (int)rank * half, bar);
                }
            }
            if (*abort_flag) {
                // copies already issued still write shared memory: the even CTA waits (bounded) for the stages it
                // announced; its partner, whose copies complete over there, stays for as long before the closing barrier
                for (int i = max(0, it - STAGES); i < it; i++)
                    for (uint32_t w = 0; w < XR_SPIN_LIMIT && (rank != 0 || !mbar_try_wait(&full[i % STAGES], (i / STAGES) & 1)); w++) {}
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (even CTA only) ----------------
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = instr_desc_pair(p.bn);
            bool ok = true;
            int it = 0, j = 0;                               // K blocks and tiles done so far
            for (int item = cluster_id; item < p.pair_tiles * p.splits && ok; item += n_clusters, j++) {
                const int split = item / p.pair_tiles;
                const int kb0 = (int)(((long long)split * nkb) / p.splits), kb1 = (int)(((long long)(split + 1) * nkb) / p.splits);
                const int b = j % ACC_BUFS;
                if (j >= ACC_BUFS) {                         // the epilogues of both CTAs have emptied this accumulator
                    ok = mbar_wait(&acc_empty[b], ((j / ACC_BUFS) - 1) & 1, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                }
                const uint32_t acc_addr = tmem_base + (uint32_t)b * TC2_BN;
                for (int i = kb0; i < kb1; i++, it++) {
                    int s = it % STAGES;
                    ok = mbar_wait(&full[s], (it / STAGES) & 1, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
                    uint32_t b_addr = a_addr + W_BYTES;
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; k++)
                        tc_mma_pair(acc_addr, smem_desc_sw128(a_addr + k * 32), smem_desc_sw128(b_addr + k * 32), idesc, (i > kb0 || k > 0) ? 1u : 0u);
                    tc_commit_pair(&empty[s]);
                }
                if (ok) tc_commit_pair(&acc_full[b]);
            }
        }
    } else {
        // ---------------- epilogue: warps 2..17 of both CTAs, each CTA its own 128 rows ----------------
        const uint32_t acc_empty_bar0 = tc_map_to_rank(smem_u32(&acc_empty[0]), 0);
        int j = 0;
        for (int item = cluster_id; item < p.pair_tiles * p.splits; item += n_clusters, j++) {
            const int tile = item % p.pair_tiles, split = item / p.pair_tiles;
            const int b = j % ACC_BUFS;
            if (!mbar_wait(&acc_full[b], (j / ACC_BUFS) & 1, abort_flag)) break;
            tc_fence_after();
            const int row0 = (2 * (tile / p.tok_tiles) + (int)rank) * TC_BM, tok0 = (tile % p.tok_tiles) * p.bn;
            tc_epilogue(p, tmem_base + (uint32_t)b * TC2_BN, row0, tok0, warp, lane, 4, split);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(acc_empty_bar0 + (uint32_t)b * 8);
        }
    }
    __syncwarp();
    tc_fence_before();
    tc_cluster_sync();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, 1);
}

// ---------------------------------------------------------------------------------------------
// Finish of a split-K product: sum the partials in split order, then the same epilogues.
// ---------------------------------------------------------------------------------------------
struct FinishParams {
    const float* partial; void* out; const float* bias;
    long long ldo;
    int n, n_out, splits, epilogue, out_dtype, gated, act;
};

__global__ void k_splitk_finish(FinishParams p) {
    xr_pdl_launch();
    xr_pdl_wait();
    size_t total = (size_t)p.n * p.n_out;
    // a gated product's partials are rows as packed: feature f has its gate row at 128 (f / 64) + 32 ((f % 64) / 16)
    // + f % 16 and its up row sixteen further
    size_t width = p.gated ? (size_t)((p.n_out + 63) / 64) * 128 : (size_t)p.n_out;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        size_t t = i / p.n_out, r = i % p.n_out;
        const size_t rg = p.gated ? (r >> 6) * 128 + ((r & 63) >> 4) * 32 + (r & 15) : r;
        const size_t ru = p.gated ? rg + 16 : rg;
        // four splits' loads in flight together (indices clamped: no load is conditional), summed in split order
        float g = 0.f, u = 0.f;
        for (int s0 = 0; s0 < p.splits; s0 += 4) {
            float a[4], b[4];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float* src = p.partial + ((size_t)min(s0 + q, p.splits - 1) * p.n + t) * width;
                a[q] = xr_ld_now(src + rg);
                b[q] = xr_ld_now(src + ru);
            }
#pragma unroll
            for (int q = 0; q < 4; q++) { xr_ld_fence(a[q]); xr_ld_fence(b[q]); }
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const bool live = s0 + q < p.splits;
                g += live ? a[q] : 0.f;
                u += (live && p.gated) ? b[q] : 0.f;
            }
        }
        float v;
        if (p.gated) v = tc_act(p.act, g) * u;
        else if (p.epilogue == TC_EPI_ADD) v = g + (p.bias ? p.bias[r] : 0.f);
        else v = tc_act(p.act, g + (p.bias ? p.bias[r] : 0.f));
        size_t o = t * p.ldo + r;
        if (p.epilogue == TC_EPI_ADD) ((float*)p.out)[o] += v;
        else if (p.out_dtype == XR_BF16) ((__nv_bfloat16*)p.out)[o] = __float2bfloat16_rn(v);
        else ((float*)p.out)[o] = v;
    }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)ptr;
    }
    return fn;
}

// [rows, K] bfloat16, row stride `ld` elements; box = 64 (K) x box_rows; 128-byte swizzle; zero fill outside.
static bool make_map(CUtensorMap* m, const void* base, long long rows, long long K, long long ld, int box_rows) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return false;
    const XrMapKey key{base, {(unsigned long long)K, (unsigned long long)rows, 0}, {(unsigned long long)ld * 2, 0}, {TC_BK, (unsigned)box_rows, 0}, 2, 0};
    return xr_cached_map(m, key, [&](CUtensorMap* out) {
        cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
        cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
        cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
        cuuint32_t estr[2] = {1, 1};
        return enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    });
}

template <int BN, int STAGES, int MINB>
static int launch_tc(const CUtensorMap& mw, const CUtensorMap& mx, const TcParams& p, dim3 grid, cudaStream_t stream) {
    constexpr int STAGE_BYTES = TC_BM * TC_BK * 2 + BN * TC_BK * 2;
    constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + (2 * STAGES + 1) * 8 + 16;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(k_gemm_tc<BN, STAGES, MINB>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
            return XR_ERR_LAUNCH;
        configured = true;
    }
    xr_launch((k_gemm_tc<BN, STAGES, MINB>), dim3(grid), dim3(tc_threads(BN)), SMEM, stream, mw, mx, p);
    return xr_launch_status();
}

#define TC2_STAGES 6
struct PairLaunch {
    static constexpr int STAGE_BYTES = TC_BM * TC_BK * 2 + (TC2_BN / 2) * TC_BK * 2;
    static constexpr int SMEM = TC2_STAGES * STAGE_BYTES + 1024 + (2 * TC2_STAGES + 4) * 8 + 16;
    static void config(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, int clusters, cudaStream_t stream) {
        cfg = {};
        cfg.gridDim = dim3(2 * clusters); cfg.blockDim = dim3(TC2_THREADS); cfg.dynamicSmemBytes = SMEM; cfg.stream = stream;
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = xr_pdl_enabled() ? 2 : 1;
    }
    // pairs of CTAs the device holds at once (one CTA per SM); 0 if it cannot run the kernel as clusters of two
    static int clusters() {
        static int n = -1;
        if (n < 0) {
            n = 0;
            cudaLaunchConfig_t cfg; cudaLaunchAttribute attr[2];
            config(cfg, attr, xr_sm_count() / 2, nullptr);
            cfg.numAttrs = 1;
            int nc = 0;
            if (cudaFuncSetAttribute(k_gemm_tc_pair<TC2_STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) == cudaSuccess &&
                cudaOccupancyMaxActiveClusters(&nc, k_gemm_tc_pair<TC2_STAGES>, &cfg) == cudaSuccess && nc > 0)
                n = nc;
            else
                cudaGetLastError();        // the single-CTA kernel takes over; leave no error behind
        }
        return n;
    }
    static int launch(const CUtensorMap& mw, const CUtensorMap& mx, const TcParams& p, cudaStream_t stream) {
        const int most = clusters();
        if (most < 1) return XR_ERR_LAUNCH;
        cudaLaunchConfig_t cfg; cudaLaunchAttribute attr[2];
        const int items = p.pair_tiles * p.splits;
        config(cfg, attr, items < most ? items : most, stream);
        cudaLaunchKernelEx(&cfg, k_gemm_tc_pair<TC2_STAGES>, mw, mx, p);
        return xr_launch_status();
    }
};

// CTAs of one product that fit the machine at once: the shared memory of the token tiles up to 64 is sized for
// two per SM (three for the 16-token tile, of which the grids fill two), one otherwise.
static int resident_ctas(int bn, int sms) { return bn <= 64 ? 2 * sms : sms; }

// Tokens per tile for a kernel whose buffers hold `cap` of them: up to `cap` tokens, the tokens rounded up to the
// instruction's step of 16 (no work on padding); more, `cap` -- narrower tiles that would fill the last wave
// better were measured (144..240 at 2,048 tokens) and are no faster, the product being bound by the operand
// traffic of its tiles rather than by the number of waves.  The width changes nothing in the sums: every
// output element is one accumulator over all of K.
static int choose_token_tile(int n, int cap) {
    if (n <= cap) return (n + 15) / 16 * 16;
    return cap;
}

// How a product is cut into work: which kernel, how wide its token tiles, how many slices along K.  One function
// for every entry point, so that two entry points given the same sizes and the same room for partial sums do the
// same arithmetic.
//
// Costs are in units of the time one CTA needs for one K block (about 0.27 us).  A product runs in waves of
// `slots` CTAs (CTA pairs in the pair kernel); a CTA costs a fixed part (launch, barrier and tensor-memory set-up,
// filling the pipeline, the epilogue: about six units) plus its K blocks.  A product that is cut along K also pays
// for its partial sums' way to memory and back (8 bytes per element and slice at about 5 TB/s, 170,000 elements a
// unit in the pair kernel, whose partial sums are tens of megabytes; a quarter of that in the single-CTA kernel, whose
// few megabytes stay in L2) and for the kernel that sums them (fifteen units; none when the caller's next kernel does
// it in passing).
// The cheapest number of slices is taken; only products with a single tile of tokens are cut (single-CTA kernel).
struct TcPlan {
    int bn;            // token capacity of the kernel's tile: 16, 32, 64, 128 or 256
    int bn_eff;        // tokens per tile as launched
    int tok_tiles, row_tiles, total_kb, splits;
    bool pair;
    long long rows;    // rows of the product (gated: 128 per 64 features)
};

static TcPlan plan_product(int n, int n_out, int K, bool gated, int force_splits, bool deferred, long long scratch_floats) {
    TcPlan pl{};
    pl.bn = n <= 16 ? 16 : (n <= 32 ? 32 : (n <= 64 ? 64 : (n <= 128 ? 128 : 256)));
    pl.row_tiles = gated ? (n_out + 63) / 64 : (n_out + TC_BM - 1) / TC_BM;
    pl.rows = gated ? (long long)pl.row_tiles * TC_BM : n_out;
    pl.total_kb = (K + TC_BK - 1) / TC_BK;
    pl.bn_eff = choose_token_tile(n, pl.bn);
    pl.tok_tiles = (n + pl.bn_eff - 1) / pl.bn_eff;
    const long long per_slice = (long long)n * pl.rows;              // partial sums of one slice
    // (the single-CTA kernel's partial sums are a few megabytes that the kernel after it finds in L2, and a deferred
    // sum rides in a kernel that runs anyway: measured at 64 tokens, charging them the pair kernel's rates picks five
    // slices for the 4096 x 4096 product where eight are faster, 9.3 against 7.7 us)
    const long long finish = deferred ? 0 : 15;
    const int pair_clusters = pl.bn == 256 ? PairLaunch::clusters() : 0;
    pl.pair = pair_clusters > 0;
    int splits = 1, max_s;
    long long tiles, slots;
    if (pl.pair) {
        pl.bn_eff = (pl.bn_eff + 31) / 32 * 32;
        pl.tok_tiles = (n + pl.bn_eff - 1) / pl.bn_eff;
        tiles = (long long)pl.tok_tiles * ((pl.row_tiles + 1) / 2);
        slots = pair_clusters;
        max_s = tiles < slots ? (pl.total_kb / 8 < 8 ? pl.total_kb / 8 : 8) : 1;
    } else {
        tiles = (long long)pl.row_tiles * pl.tok_tiles;
        slots = resident_ctas(pl.bn, xr_sm_count());
        max_s = (pl.tok_tiles > 1 || tiles >= 2 * slots) ? 1 : (pl.total_kb / 4 < 16 ? pl.total_kb / 4 : 16);
    }
    if (max_s < 1) max_s = 1;
    if (force_splits > 0) splits = force_splits;
    else {
        long long best_cost = -1;
        for (int sp = 1; sp <= max_s; sp++) {
            long long rounds = (tiles * sp + slots - 1) / slots;
            long long cost = rounds * (6 + (pl.total_kb + sp - 1) / sp);
            if (sp > 1) cost += pl.pair ? finish + sp * per_slice / 170000 : finish + sp * per_slice / 700000;
            if (best_cost < 0 || cost < best_cost) { best_cost = cost; splits = sp; }
        }
    }
    if (splits > pl.total_kb) splits = pl.total_kb;
    // no room for the partial sums: the product runs uncut (slower, the same result up to the order of the sums)
    if (splits > 1 && scratch_floats < (long long)splits * per_slice) splits = 1;
    pl.splits = splits;
    return pl;
}

// Room for partial sums that no product of these sizes exceeds.
XR_EXPORT long long xr_gemm_tc_scratch_floats(int n, int n_out, int gated) {
    return 16LL * (long long)n * (gated ? (long long)((n_out + 63) / 64) * 128 : (long long)n_out);
}

// X: [n, K] bfloat16 (row stride ldx).  W: [n_out, K] bfloat16 dense, or packed tile by tile
// ([row tile][K block][128][64], rows and K padded with zeros to whole tiles; n_out is then the logical row count).
// epilogue: TC_EPI_STORE / TC_EPI_ADD / TC_EPI_GATED; act: TC_ACT_* (store: on the stored value; gated: on the gate).
// A gated product needs the packed layout with gate and up rows interleaved (every 128-row tile holds 64 features:
// in each quarter sixteen gate rows, then their sixteen up rows); n_out counts features and out is [n, n_out].
// scratch: float32 workspace for products cut along K (xr_gemm_tc_scratch_floats bounds what is used); status:
// device int, set non-zero if a wait gave up.
XR_EXPORT int xr_gemm_tc(const void* X, const void* W, const float* bias, void* out, int out_dtype, int epilogue, int act,
                         int n, int n_out, int K, long long ldx, long long ldo, float* scratch,
                         long long scratch_floats, int* status, int force_splits, int defer_finish, int* splits_used,
                         int w_packed, cudaStream_t stream) {
    if (n < 1 || n_out < 1 || K < 8 || (K % 8) != 0 || (ldx % 8) != 0 || ldx < K || ldo < n_out) return XR_ERR_ARG;
    if (((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return XR_ERR_ARG;
    if (epilogue != TC_EPI_STORE && epilogue != TC_EPI_ADD && epilogue != TC_EPI_GATED) return XR_ERR_ARG;
    if (epilogue == TC_EPI_ADD && (out_dtype != XR_F32 || act != TC_ACT_NONE)) return XR_ERR_ARG;
    if (out_dtype != XR_F32 && out_dtype != XR_BF16) return XR_ERR_ARG;
    if (act != TC_ACT_NONE && act != TC_ACT_SILU && act != TC_ACT_GELU_TANH) return XR_ERR_ARG;
    const bool gated = epilogue == TC_EPI_GATED;
    if (gated && (!w_packed || bias != nullptr)) return XR_ERR_ARG;
    const TcPlan pl = plan_product(n, n_out, K, gated, force_splits, defer_finish != 0, scratch ? scratch_floats : 0);
    CUtensorMap mw, mx;
    const int rows_padded = gated ? (int)pl.rows : (n_out + TC_BM - 1) / TC_BM * TC_BM;
    if (w_packed) {
        if (!make_map(&mw, W, (long long)rows_padded * pl.total_kb, TC_BK, TC_BK, TC_BM)) return -3;
    } else if (!make_map(&mw, W, n_out, K, K, TC_BM)) return -3;
    if (!make_map(&mx, X, n, K, ldx, pl.pair ? pl.bn_eff / 2 : pl.bn_eff)) return -3;
    const int splits = pl.splits;
    if (pl.row_tiles > 65535 || splits > 65535) return XR_ERR_ARG;
    if (splits_used) *splits_used = splits;
    TcParams p{out, bias, scratch, status, ldo, n, n_out, K, splits, splits > 1 ? TC_EPI_PARTIAL : epilogue, out_dtype,
               act, gated ? 1 : 0, pl.bn_eff, w_packed, pl.total_kb, pl.tok_tiles, pl.tok_tiles * ((pl.row_tiles + 1) / 2)};
    dim3 grid(pl.tok_tiles, pl.row_tiles, splits);
    int rc;
    if (pl.pair) {
        rc = PairLaunch::launch(mw, mx, p, stream);
    } else {
        // With no more CTAs than SMs a CTA has its SM to itself: a ring twice as deep keeps as many bytes in flight as two
        // CTAs would (the gated product of Llama-3.2-1B layer sizes at 64 tokens, 128 uncut tiles: 17.6 -> 15.9 us inside a
        // step; what is left to the 10 us of its bytes is the tokens' tile, which every CTA fetches again with each
        // K block through the same copy engine as its weights).
        const bool alone = (long long)pl.tok_tiles * pl.row_tiles * splits <= xr_sm_count();
        switch (pl.bn) {
            case 16: rc = launch_tc<16, 4, 3>(mw, mx, p, grid, stream); break;
            case 32: rc = alone ? launch_tc<32, 10, 1>(mw, mx, p, grid, stream) : launch_tc<32, 5, 2>(mw, mx, p, grid, stream); break;
            case 64: rc = alone ? launch_tc<64, 8, 1>(mw, mx, p, grid, stream) : launch_tc<64, 4, 2>(mw, mx, p, grid, stream); break;
            case 128: rc = launch_tc<128, 5, 1>(mw, mx, p, grid, stream); break;
            default: rc = launch_tc<256, 4, 1>(mw, mx, p, grid, stream); break;
        }
    }
    if (rc != XR_OK || splits == 1 || defer_finish) return rc;      // deferred: the caller's next kernel sums the partials
    FinishParams f{scratch, out, bias, ldo, n, n_out, splits, epilogue, out_dtype, gated ? 1 : 0, act};
    size_t total = (size_t)n * n_out;
    const int most = xr_sm_count() * 8;
    int blocks = (int)((total + 255) / 256 < (size_t)most ? (total + 255) / 256 : most);
    xr_launch(k_splitk_finish, dim3(blocks), dim3(256), 0, stream, f);
    return xr_launch_status();
}

// ---------------------------------------------------------------------------------------------
// An entry point that allocates nothing (declared in xrb200_noalloc.h; it has no counterpart in the
// reference).  Same product as xr_gemm_tc, but the split-K scratch and the status word live in arrays
// that are part of this library's image, so the caller passes inputs and outputs only.
//
// In host code the names below stand for the arrays but are not device addresses; the address a kernel
// can use comes from cudaGetSymbolAddress, asked once per device (with that device current) on the
// entry point's first call there.
// ---------------------------------------------------------------------------------------------
#define XR_NOALLOC_SCRATCH_FLOATS (4u << 20)          // 16 MiB of float32, held by every GPU that loads the library
#define XR_NOALLOC_MAX_DEVICES 64
static __device__ __align__(256) float g_noalloc_scratch[XR_NOALLOC_SCRATCH_FLOATS];
static __device__ __align__(256) int g_noalloc_status[64];

static float* g_noalloc_scratch_ptr[XR_NOALLOC_MAX_DEVICES];
static int* g_noalloc_status_ptr[XR_NOALLOC_MAX_DEVICES];

XR_EXPORT long long xr_gemm_tc_noalloc_max_floats() { return (long long)XR_NOALLOC_SCRATCH_FLOATS; }

XR_EXPORT int xr_gemm_tc_noalloc(const void* X, const void* W, const float* bias, void* out, int out_dtype, int epilogue,
                                 int n, int n_out, int K, long long ldx, long long ldo, int* status_out_host,
                                 cudaStream_t stream) {
    // arguments first: nothing is queued for a call that is refused
    if (n < 1 || n_out < 1 || K < 8 || (K % 8) != 0 || (ldx % 8) != 0 || ldx < K || ldo < n_out) return XR_ERR_ARG;
    if (((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return XR_ERR_ARG;
    if (epilogue != TC_EPI_STORE && epilogue != TC_EPI_ADD) return XR_ERR_ARG;        // (the gated product wants packed weights)
    if ((out_dtype != XR_F32 && out_dtype != XR_BF16) || (epilogue == TC_EPI_ADD && out_dtype != XR_F32)) return XR_ERR_ARG;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= XR_NOALLOC_MAX_DEVICES) return -5;
    if (g_noalloc_scratch_ptr[dev] == nullptr) {
        // set-up, once per device: resolve the arrays' device addresses
        float* sp = nullptr; int* st = nullptr;
        if (cudaGetSymbolAddress((void**)&sp, g_noalloc_scratch) != cudaSuccess || sp == nullptr) return -5;
        if (cudaGetSymbolAddress((void**)&st, g_noalloc_status) != cudaSuccess || st == nullptr) return -5;
        g_noalloc_status_ptr[dev] = st;
        g_noalloc_scratch_ptr[dev] = sp;
    }
    // The cut that the ordinary entry point makes when it has all the room it may want; if the fixed array is too
    // small for it the call is refused rather than run with another cut (and other rounding) than the caller expects.
    const TcPlan want = plan_product(n, n_out, K, false, 0, false, xr_gemm_tc_scratch_floats(n, n_out, 0));
    if (want.splits > 1 && (long long)want.splits * n * n_out > (long long)XR_NOALLOC_SCRATCH_FLOATS) return -4;
    // the status word must start at zero; the scratch needs no clearing (every partial that is read was
    // written by this call first)
    if (cudaMemsetAsync(g_noalloc_status_ptr[dev], 0, sizeof(int), stream) != cudaSuccess) return XR_ERR_LAUNCH;
    int rc = xr_gemm_tc(X, W, bias, out, out_dtype, epilogue, TC_ACT_NONE, n, n_out, K, ldx, ldo, g_noalloc_scratch_ptr[dev],
                        (long long)XR_NOALLOC_SCRATCH_FLOATS, g_noalloc_status_ptr[dev], want.splits, 0, nullptr, 0, stream);
    if (rc != XR_OK) return rc;
    if (status_out_host != nullptr) {
        // optional: wait for the product and report whether a wait inside it gave up
        if (cudaMemcpyAsync(status_out_host, g_noalloc_status_ptr[dev], sizeof(int), cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
            cudaStreamSynchronize(stream) != cudaSuccess)
            return XR_ERR_LAUNCH;
    }
    return XR_OK;
}
