// Causal grouped-query attention of prompt portions on the 5th-generation tensor cores (tcgen05), over the
// paged cache: S = Q K^T and O += P V as tcgen05.mma with S and O in tensor memory, Q, K, V brought to shared
// memory by TMA (128-byte swizzle; K and V straight from the pages), softmax in float32 by the thread that
// owns the row.  Same arithmetic as the row-tiled mma.sync kernel (attention_mma.cu), which stays as the
// path for the shapes this one does not take.  Needs bfloat16, head size 64 or 128 (one or two 64-column
// halves of Q, K, V and O), heads per kv head dividing 128, a power-of-two page size >= 8.
//
// A CTA owns 128 packed rows (token i / G, head i % G) of one (request, kv head) and walks its keys in tiles
// of 128, in ascending order.  Roles (352 threads):
//   warps 0..7 : softmax.  Row r = tensor-memory lane r is shared by two threads (warps w and w + 4 may both
//                read lanes 32 (w % 4) ..): one takes keys 0..63 of a tile, the other keys 64..127; they
//                exchange their maxima through shared memory.  Per tile: read S, running maximum, rescale O in
//                tensor memory when needed, write P = exp(S - m) as bfloat16 over the first 64 columns of the
//                tile's own S in tensor memory (row = lane, two values per column), where the product reads it
//                as its A operand (half the shared-memory traffic of P V against P passed through shared memory, and
//                no stores of P there).  One softmax warp per scheduler could not hide its own latencies; two can.
//   warp 8     : one lane issues the TMA copies of Q (once) and of the K tiles (two-stage ring; a K stage is free
//                as soon as its Q K^T has run, so the next-but-one tile's keys are fetched two tiles ahead).
//   warp 9     : one lane issues the matrix instructions; the warp owns the tensor-memory allocation.
//   warp 10    : one lane issues the TMA copies of the V tiles (two-stage ring, freed by P V).
// S (and with it P) is double buffered (S of tile j+1 is computed, and P of tile j is consumed, while the softmax
// of the neighbouring tile runs); O is one accumulator.  O and the running sum carry an offset m per row; the offset
// is moved (and O rescaled, which has to wait for the product in flight) only when a row's maximum has grown by
// more than 8 (in log2) since it was set, so most tiles never wait: exp2(s - m) then stays below 2^8.
// V is the B operand of P V with N = head size contiguous in memory (an "MN-major" operand): its shared
// memory descriptor has leading byte offset = distance between the two 64-column halves and stride byte
// offset = 8 keys.
//
// Every wait is bounded; a wait that runs out is recorded in the status word and the CTA runs on (its
// output is then meaningless) so that all its threads still meet at the barriers and tensor memory is freed.
//
// The reference computes prompt attention with one block per (head, token) and a global score scratch
// (`k_attn`, src/kernels.cu:2043-2141); formulas src/model.c:3548-3589, 3409-3415.
#include "common.cuh"
#include <cuda.h>
#include <math.h>

#define TA_ROWS 128
#define TA_KEYS 128
#define TA_THREADS 352
#define TA_SPIN (1u << 24)

struct AttnTcArgs {
    __nv_bfloat16* out;          // [n, H * hd]
    const int* seg_start; const int* seg_len; const int* seg_pos0; const int* block_tables;
    int* status;
    int H, K, G, max_pages, page_size, page_shift, window, n_layers, layer;
    float scale_log2;            // scale * log2(e)
    int n_seg;
};

__device__ __forceinline__ uint32_t ta_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ta_bar_init(uint64_t* b, uint32_t n) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ta_smem(b)), "r"(n)); }
__device__ __forceinline__ void ta_expect(uint64_t* b, uint32_t bytes) { asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(ta_smem(b)), "r"(bytes) : "memory"); }
__device__ __forceinline__ void ta_arrive(uint64_t* b) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ta_smem(b)) : "memory"); }
__device__ __forceinline__ void ta_wait(uint64_t* b, uint32_t parity, volatile int* gave_up) {
    for (uint32_t i = 0; i < TA_SPIN; i++) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(ta_smem(b)), "r"(parity) : "memory");
        if (ok) return;
        if ((i & 4095u) == 4095u && *gave_up) return;
    }
    *gave_up = 1;
}
__device__ __forceinline__ void ta_tma_2d(void* dst, const CUtensorMap* m, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(ta_smem(dst)), "l"(m), "r"(x), "r"(y), "r"(ta_smem(bar)) : "memory");
}
__device__ __forceinline__ void ta_tma_3d(void* dst, const CUtensorMap* m, int x, int y, int z, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(ta_smem(dst)), "l"(m), "r"(x), "r"(y), "r"(z), "r"(ta_smem(bar)) : "memory");
}
__device__ __forceinline__ void ta_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(ta_smem(bar)) : "memory");
}
__device__ __forceinline__ void ta_mma(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
// the same with the A operand in tensor memory: row = lane, two bfloat16 per 32-bit column, K along the columns
__device__ __forceinline__ void ta_mma_ts(uint32_t d, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(d), "r"(a_tmem), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void ta_ld32(uint32_t taddr, float* v) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}
// the same load without the wait, so that several can be in flight; call ta_ld_wait() before using the values
__device__ __forceinline__ void ta_ld32_nowait(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void ta_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void ta_st32(uint32_t taddr, const float* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
          "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
          "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
          "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
          "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
          "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
          "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
          "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
}
__device__ __forceinline__ void ta_st32u(uint32_t taddr, const uint32_t* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
          "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]),
          "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]),
          "r"(v[30]), "r"(v[31])
        : "memory");
}
__device__ __forceinline__ float ta_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// K-major operand (rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart)
__device__ __forceinline__ uint64_t ta_desc_k(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// MN-major operand: 64 contiguous N elements per 128-byte row, rows are K (keys), 8-key groups 1024 bytes
// apart (stride byte offset), the next 64 N elements `lbo` bytes on (leading byte offset)
__device__ __forceinline__ uint64_t ta_desc_mn(uint32_t saddr, uint32_t lbo) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// instruction descriptor: float32 accumulate, bfloat16 A and B, M = 128, N = n; b_mn: B is MN-major
__host__ __device__ constexpr uint32_t ta_idesc(bool b_mn, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

// HD: head size, 64 or 128.  Shared memory keeps the layout of head size 128 (a stage of K or V is two halves
// apart); at head size 64 only the first half of each is filled and read.
template <int HD>
__global__ void __launch_bounds__(TA_THREADS, 1)
k_attention_tc(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map, AttnTcArgs a) {
    // 10 half tiles of 16 KB; the array is declared 1 KB aligned (what the
    // swizzled TMA boxes and the matrix descriptors need) and the kernel refuses to run if it is not
    extern __shared__ __align__(1024) uint8_t ta_smem_raw[];
    uint8_t* smem = ta_smem_raw;
    if ((ta_smem(smem) & 1023u) != 0) {
        if (threadIdx.x == 0) atomicExch(a.status, 4);
        return;
    }
    constexpr int HALF = TA_ROWS * 128;                   // bytes of one [128 rows][64 columns] half tile
    constexpr int NH = HD / 64;                           // 64-column halves of a head
    static_assert(HD == 64 || HD == 128, "head size 64 or 128");
    uint8_t* q_s = smem;                                  // [2 halves][128 rows][128 B]
    uint8_t* k_s = q_s + 2 * HALF;                        // [2 stages][2 halves (hd)][128 keys][128 B]
    uint8_t* v_s = k_s + 4 * HALF;                        // [2 stages][2 halves (hd)][128 keys][128 B]
    uint64_t* bars = (uint64_t*)(v_s + 4 * HALF);
    uint64_t* q_full = bars;            // 1
    uint64_t* k_full = bars + 1;        // 2
    uint64_t* v_full = bars + 3;        // 2
    uint64_t* k_empty = bars + 5;       // 2
    uint64_t* s_full = bars + 7;        // 2
    uint64_t* p_full = bars + 9;        // 1  (count 8)
    uint64_t* pv_done = bars + 10;      // 2  (product of tile j arrives on pv_done[j & 1]; it also frees V stage j & 1)
    uint32_t* tmem_slot = (uint32_t*)(bars + 12);
    volatile int* gave_up = (volatile int*)(tmem_slot + 1);
    float* xch = (float*)(tmem_slot + 4);                // [2 tile parities][2 key halves][128 rows]

    // The row tiles of the portions with more than 16 packed rows, laid end to end, are the grid's x (short portions
    // belong to the key-split kernel and have no blocks here: a step may hold dozens of them beside one prompt
    // portion).  A block finds its (portion, tile) by walking the portions' lengths; later tiles, which have the most
    // keys, start first.
    const int kvh = blockIdx.y;
    int seg = -1, tile = 0;
    {
        const int want = (int)gridDim.x - 1 - (int)blockIdx.x;
        int before = 0;
        for (int s = 0; s < a.n_seg; s++) {
            const int rows = a.seg_len[s] * a.G;
            const int t = rows > 16 ? (rows + TA_ROWS - 1) / TA_ROWS : 0;
            if (want < before + t) { seg = s; tile = want - before; break; }
            before += t;
        }
    }
    if (seg < 0) return;                                            // (the caller gave an upper bound of the tiles)
    const int L = a.seg_len[seg], rows_total = L * a.G;
    const int row0 = tile * TA_ROWS;
    xr_pdl_launch();
    xr_pdl_wait();
    const int pos0 = a.seg_pos0[seg], tok_base = a.seg_start[seg];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int last_row = min(rows_total, row0 + TA_ROWS) - 1;
    const int hi = pos0 + last_row / a.G;
    const int lo = a.window > 0 ? max(0, pos0 + row0 / a.G - a.window + 1) : 0;
    const int t_lo = lo / TA_KEYS, t_hi = hi / TA_KEYS, n_tiles = t_hi - t_lo + 1;

    if (threadIdx.x == 0) {
        ta_bar_init(q_full, 1);
        for (int i = 0; i < 2; i++) { ta_bar_init(&k_full[i], 1); ta_bar_init(&v_full[i], 1); ta_bar_init(&k_empty[i], 1); ta_bar_init(&s_full[i], 1); }
        ta_bar_init(p_full, 8);            // one arrival per softmax warp
        ta_bar_init(&pv_done[0], 1);
        ta_bar_init(&pv_done[1], 1);
        *gave_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ta_smem(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    const uint32_t tm_s0 = tmem, tm_s1 = tmem + 128, tm_o = tmem + 256;

    if (warp == 8 || warp == 10) {
        // ---------------- TMA producers: warp 8 Q and K, warp 10 V ----------------
        if (lane == 0) {
            const bool keys = warp == 8;
            if (keys) {
                ta_expect(q_full, NH * HALF);
                int tok0 = tok_base + row0 / a.G;
                for (int c = 0; c < NH; c++) ta_tma_3d(q_s + c * HALF, &q_map, c * 64, kvh * a.G, tok0, q_full);
            }
            const int box_rows = a.page_size < 64 ? a.page_size : 64;
            uint64_t* full = keys ? k_full : v_full;
            uint64_t* empty = keys ? k_empty : pv_done;
            uint8_t* base = keys ? k_s : v_s;
            for (int j = 0; j < n_tiles; j++) {
                int s = j & 1;
                if (j >= 2) ta_wait(&empty[s], ((j >> 1) - 1) & 1, gave_up);
                ta_expect(&full[s], NH * HALF);
                int key0 = (t_lo + j) * TA_KEYS;
                for (int r0 = 0; r0 < TA_KEYS; r0 += box_rows) {
                    int kp = key0 + r0;
                    int pi = kp >> a.page_shift;
                    int page = pi < a.max_pages ? a.block_tables[(size_t)seg * a.max_pages + pi] : -1;
                    long long row = ((((long long)page * a.n_layers + a.layer) * 2 + (keys ? 0 : 1)) * a.K + kvh) * a.page_size + (kp & (a.page_size - 1));
                    if (page < 0) row = -1024;                          // outside the tensor: the copy fills zeros
                    for (int c = 0; c < NH; c++) ta_tma_2d(base + (s * 2 + c) * HALF + r0 * 128, &kv_map, c * 64, (int)row, &full[s]);
                }
            }
        }
    } else if (warp == 9) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t id_qk = ta_idesc(false, TA_KEYS), id_pv = ta_idesc(true, HD);
            auto issue_qk = [&](int j) {
                int s = j & 1;
                ta_wait(&k_full[s], (j >> 1) & 1, gave_up);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                uint32_t qa = ta_smem(q_s), kb = ta_smem(k_s + s * 2 * HALF);
#pragma unroll
                for (int kk = 0; kk < HD / 16; kk++) {
                    uint32_t off = (kk >> 2) * HALF + (kk & 3) * 32;
                    ta_mma((j & 1) ? tm_s1 : tm_s0, ta_desc_k(qa + off), ta_desc_k(kb + off), id_qk, kk > 0 ? 1u : 0u);
                }
                ta_commit(&s_full[j & 1]);
                ta_commit(&k_empty[s]);          // the keys of this tile are not needed again
            };
            ta_wait(q_full, 0, gave_up);
            issue_qk(0);
            for (int j = 0; j < n_tiles; j++) {
                int s = j & 1;
                // S of the next tile while the softmax of this one runs: its buffer was released by p_full(j-1),
                // which this thread waited for in the previous round
                if (j + 1 < n_tiles) issue_qk(j + 1);
                ta_wait(p_full, j & 1, gave_up);                    // P(j) is in tensor memory, S(j) has been read
                ta_wait(&v_full[s], (j >> 1) & 1, gave_up);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                uint32_t vb = ta_smem(v_s + s * 2 * HALF);
                const uint32_t tm_p = (j & 1) ? tm_s1 : tm_s0;
#pragma unroll
                for (int kk = 0; kk < TA_KEYS / 16; kk++) {
                    uint64_t bd = ta_desc_mn(vb + kk * 16 * 128, HALF);
                    ta_mma_ts(tm_o, tm_p + kk * 8, bd, id_pv, (j > 0 || kk > 0) ? 1u : 0u);
                }
                ta_commit(&pv_done[j & 1]);
            }
        }
    } else {
        // ---------------- softmax: row = tensor-memory lane, two threads per row (key halves) ----------------
        const int r = (warp & 3) * 32 + lane;                    // 0..127
        const int half = warp >> 2;                              // keys [64 half, 64 half + 64) of every tile
        const int pr = row0 + r;
        const int pos = pr < rows_total ? pos0 + pr / a.G : -1;
        const int lo_r = a.window > 0 ? pos - a.window + 1 : 0;
        const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
        float m = -INFINITY, l = 0.f;          // m: the offset O and l currently carry (log2 domain); l: this thread's half
        const int pos_first = pos0 + row0 / a.G;                  // smallest position of the CTA's rows
        for (int j = 0; j < n_tiles; j++) {
            const uint32_t tm_s = ((j & 1) ? tm_s1 : tm_s0) + lane_off + half * 64;
            const int key0 = (t_lo + j) * TA_KEYS + half * 64;
            // a tile every row sees whole needs no per-score mask
            const bool masked = a.window > 0 || (t_lo + j) * TA_KEYS + TA_KEYS - 1 > pos_first || row0 + TA_ROWS > rows_total;
            ta_wait(&s_full[j & 1], (j >> 1) & 1, gave_up);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // this thread's 64 scores are read once and stay in registers for both passes
            uint32_t sraw[64];
            ta_ld32_nowait(tm_s, sraw);
            ta_ld32_nowait(tm_s + 32, sraw + 32);
            ta_ld_wait();
            float v[32];
            float mx = -INFINITY;
            if (masked) {
#pragma unroll
                for (int i = 0; i < 64; i++) {
                    int kp = key0 + i;
                    if (kp <= pos && kp >= lo_r) mx = fmaxf(mx, __uint_as_float(sraw[i]));
                }
            } else {
                float m0 = __uint_as_float(sraw[0]), m1 = __uint_as_float(sraw[1]), m2 = __uint_as_float(sraw[2]), m3 = __uint_as_float(sraw[3]);
#pragma unroll
                for (int i = 4; i < 64; i += 4) {
                    m0 = fmaxf(m0, __uint_as_float(sraw[i])); m1 = fmaxf(m1, __uint_as_float(sraw[i + 1]));
                    m2 = fmaxf(m2, __uint_as_float(sraw[i + 2])); m3 = fmaxf(m3, __uint_as_float(sraw[i + 3]));
                }
                mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
            }
            // the row's maximum over both halves
            float* x = xch + (j & 1) * 256;
            x[half * 128 + r] = mx;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            mx = fmaxf(x[r], x[128 + r]) * a.scale_log2;
            // move the offset only when the maximum has grown by more than 8 since it was set
            float corr = 1.0f;
            if (m == -INFINITY) { if (mx != -INFINITY) m = mx; }          // O and l of this row are still zero
            else if (mx > m + 8.0f) { corr = ta_exp2(m - mx); m = mx; }
            if (j > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {
                // O is in use by the product of the previous tile until it completes; each thread rescales its half of the columns
                ta_wait(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, gave_up);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                l *= corr;
#pragma unroll 1
                for (int c = 0; c < NH; c++) {
                    ta_ld32(tm_o + lane_off + half * (HD / 2) + c * 32, v);
#pragma unroll
                    for (int i = 0; i < 32; i++) v[i] *= corr;
                    ta_st32(tm_o + lane_off + half * (HD / 2) + c * 32, v);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            }
            // (P lies over this tile's own S, which the tensor core wrote after the product of tile j - 2 had read its P)
            const float off = m == -INFINITY ? 0.f : m;
            // The probabilities of this thread's 64 keys.  The pass without a mask has no branch inside, so that the
            // compiler can interleave the elements' chains (scale, exp2, sum, round) instead of walking them one by one.
            float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
            uint32_t pall[32];
            if (!masked) {
#pragma unroll
                for (int i = 0; i < 64; i += 4) {
                    float p0 = ta_exp2(fmaf(__uint_as_float(sraw[i]), a.scale_log2, -off));
                    float p1 = ta_exp2(fmaf(__uint_as_float(sraw[i + 1]), a.scale_log2, -off));
                    float p2 = ta_exp2(fmaf(__uint_as_float(sraw[i + 2]), a.scale_log2, -off));
                    float p3 = ta_exp2(fmaf(__uint_as_float(sraw[i + 3]), a.scale_log2, -off));
                    sum0 += p0; sum1 += p1; sum2 += p2; sum3 += p3;
                    __nv_bfloat162 b01 = __floats2bfloat162_rn(p0, p1), b23 = __floats2bfloat162_rn(p2, p3);
                    pall[i >> 1] = *reinterpret_cast<uint32_t*>(&b01);
                    pall[(i >> 1) + 1] = *reinterpret_cast<uint32_t*>(&b23);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 64; i += 2) {
                    float p0 = ta_exp2(fmaf(__uint_as_float(sraw[i]), a.scale_log2, -off));
                    float p1 = ta_exp2(fmaf(__uint_as_float(sraw[i + 1]), a.scale_log2, -off));
                    const int kp = key0 + i;
                    p0 = (kp <= pos && kp >= lo_r) ? p0 : 0.f;
                    p1 = (kp + 1 <= pos && kp + 1 >= lo_r) ? p1 : 0.f;
                    sum0 += p0; sum1 += p1;
                    __nv_bfloat162 bb = __floats2bfloat162_rn(p0, p1);
                    pall[i >> 1] = *reinterpret_cast<uint32_t*>(&bb);
                }
            }
            sum0 = (sum0 + sum1) + (sum2 + sum3);
            // this thread's 64 probabilities, two per column, over columns 32 half .. 32 half + 31 of the tile's S
            ta_st32u(((j & 1) ? tm_s1 : tm_s0) + lane_off + half * 32, pall);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            l += sum0;
            if ((t_lo + j) * TA_KEYS + TA_KEYS - 1 > hi) {
                // The tile runs past the last key.  Probabilities there are zero, but the value rows hold whatever the
                // page held before; clear them so that zero times those bytes is zero whatever they are.
                int s = j & 1;
                ta_wait(&v_full[s], (j >> 1) & 1, gave_up);
                int first_bad = hi + 1 - (t_lo + j) * TA_KEYS;
                constexpr int CH = HD / 8;                               // 16-byte chunks of a value row
                for (int e = half * 128 + r; e < (TA_KEYS - first_bad) * CH; e += 256) {
                    int row = first_bad + e / CH, ch = e % CH;
                    *reinterpret_cast<uint4*>(v_s + (s * 2 + (ch >> 3)) * HALF + row * 128 + (((ch & 7) ^ (row & 7)) << 4)) = make_uint4(0, 0, 0, 0);
                }
            }
            // make the cleared rows visible to the tensor core (async proxy), order the tensor-memory accesses, then signal
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) ta_arrive(p_full);
        }
        ta_wait(&pv_done[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1, gave_up);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        {
            // the row's sum over both halves
            float* x = xch + (n_tiles & 1) * 256;
            x[half * 128 + r] = l;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            l = x[r] + x[128 + r];
            const bool live = pr < rows_total;
            float inv = live ? 1.0f / l : 0.f;
            __nv_bfloat16* dst = a.out + ((long long)(tok_base + (live ? pr : 0) / a.G) * a.H + (kvh * a.G + (live ? pr : 0) % a.G)) * HD + half * (HD / 2);
            float v[32];
#pragma unroll 1
            for (int c = 0; c < NH; c++) {
                ta_ld32(tm_o + lane_off + half * (HD / 2) + c * 32, v);      // warp-wide: rows past the portion load too
                if (!live) continue;
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    uint32_t w[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        __nv_bfloat162 bb = __floats2bfloat162_rn(v[i + 2 * e] * inv, v[i + 2 * e + 1] * inv);
                        w[e] = *reinterpret_cast<uint32_t*>(&bb);
                    }
                    *reinterpret_cast<uint4*>(dst + c * 32 + i) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 9) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
    if (threadIdx.x == 0 && *gave_up) atomicExch(a.status, 3);
}

// ---------------------------------------------------------------------------------------------
typedef CUresult (*TaEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static TaEncodeFn ta_encode() {
    static TaEncodeFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (TaEncodeFn)ptr;
    }
    return fn;
}

// 1 if this kernel takes the shape, 0 if not (the caller then uses the mma.sync kernel).
XR_EXPORT int xr_attention_tc_supported(int H, int K, int hd, int page_size) {
    if ((hd != 64 && hd != 128) || K < 1 || H % K != 0) return 0;
    int G = H / K;
    if (G > 128 || (128 % G) != 0) return 0;
    if (page_size < 8 || (page_size & (page_size - 1)) != 0) return 0;
    return 1;
}

// q: the step's fused rows [n, (H + 2K) * hd] (Q heads first), out: [n, H * hd].  cache_base: the cache group's
// whole array [pages][layers][K|V][kv heads][page_size][hd].  Handles the portions with more than 16 packed rows.
XR_EXPORT int xr_attention_tc(const void* q, void* out, const void* cache_base, const int* seg_start, const int* seg_len,
                              const int* seg_pos0, const int* block_tables, int* status, long long q_row_stride, int n,
                              int n_seg, int H, int K, int hd, int max_pages, int page_size, int window, float scale,
                              int max_seg_len, long long row_tiles, long long n_pages, int n_layers, int layer, cudaStream_t stream) {
    if (!xr_attention_tc_supported(H, K, hd, page_size) || n < 1 || n_seg < 1 || window < 0 || status == nullptr) return XR_ERR_ARG;
    if (((uintptr_t)q & 15) || ((uintptr_t)cache_base & 15) || (q_row_stride % 8) != 0) return XR_ERR_ARG;
    const int G = H / K;
    long long total_rows = n_pages * n_layers * 2 * K * page_size;
    if (total_rows >= (1LL << 31) || n_seg > 65535 || K > 65535) return XR_ERR_ARG;
    TaEncodeFn enc = ta_encode();
    if (!enc) return -3;
    CUtensorMap qm, kvm;
    {
        // Q as [token][head][hd]; a box is 64 columns x G heads x (128 / G) tokens = 128 packed rows
        const XrMapKey key{q, {(unsigned long long)hd, (unsigned long long)H, (unsigned long long)n}, {(unsigned long long)hd * 2, (unsigned long long)q_row_stride * 2},
                           {64, (unsigned)G, (unsigned)(TA_ROWS / G)}, 3, 0};
        if (!xr_cached_map(&qm, key, [&](CUtensorMap* out) {
                cuuint64_t dims[3] = {(cuuint64_t)hd, (cuuint64_t)H, (cuuint64_t)n};
                cuuint64_t strides[2] = {(cuuint64_t)hd * 2, (cuuint64_t)q_row_stride * 2};
                cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)(TA_ROWS / G)};
                cuuint32_t estr[3] = {1, 1, 1};
                return enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
            }))
            return -3;
    }
    {
        const unsigned box_rows = (unsigned)(page_size < 64 ? page_size : 64);
        const XrMapKey key{cache_base, {(unsigned long long)hd, (unsigned long long)total_rows, 0}, {(unsigned long long)hd * 2, 0}, {64, box_rows, 0}, 2, 1};
        if (!xr_cached_map(&kvm, key, [&](CUtensorMap* out) {
                cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)total_rows};
                cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
                cuuint32_t box[2] = {64, box_rows};
                cuuint32_t estr[2] = {1, 1};
                return enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(cache_base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
            }))
            return -3;
    }
    int shift = 0;
    while ((1 << shift) < page_size) shift++;
    AttnTcArgs a{(__nv_bfloat16*)out, seg_start, seg_len, seg_pos0, block_tables, status, H, K, G, max_pages, page_size, shift,
                 window, n_layers, layer, scale * 1.4426950408889634f, n_seg};
    constexpr int SMEM = 10 * TA_ROWS * 128 + 128 + 2 * 2 * 128 * 4;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(k_attention_tc<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess ||
            cudaFuncSetAttribute(k_attention_tc<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
            return XR_ERR_LAUNCH;
        configured = true;
    }
    // row_tiles: the 128-row tiles of the portions with more than 16 packed rows, summed; 0: not known, and an upper
    // bound is taken (blocks beyond the true number return at once)
    long long tiles = row_tiles > 0 ? row_tiles : (((long long)max_seg_len * G + TA_ROWS - 1) / TA_ROWS) * n_seg;
    if (tiles > 0x7fffffffLL) return XR_ERR_ARG;
    const dim3 grid((unsigned)tiles, K, 1);
    if (hd == 128) xr_launch(k_attention_tc<128>, grid, dim3(TA_THREADS), SMEM, stream, qm, kvm, a);
    else xr_launch(k_attention_tc<64>, grid, dim3(TA_THREADS), SMEM, stream, qm, kvm, a);
    return xr_launch_status();
}
