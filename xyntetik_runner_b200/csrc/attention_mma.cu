// Causal grouped-query attention over the paged cache on tensor cores (bfloat16 in, float32 softmax and
// accumulation), for prompt portions and for decoded tokens, head sizes 16..128 in steps of 16.
//
// For the query at position p, head h, kv head h / (H/K):  s_t = (q . k_t) * scale over the keys
// t0 <= t <= p (t0 = max(0, p - window + 1), or 0), a = softmax(s), o = sum_t a_t v_t
// (src/model.c:3548-3589, 3409-3415).  The reference's kernels are `k_attn` (one block per head and
// token, scores through a global scratch, src/kernels.cu:2043-2141) and the split `k_attn_dec` +
// `k_attn_merge` for decoding (src/kernels.cu:2171-2270).
//
// The G = H/K query heads of one kv head are packed along the M axis of the matrix instruction: packed
// row i of a request's portion is (token i / G, head i % G), so every K and V element that is loaded
// serves G heads.  Keys are walked in tiles of 64 aligned to absolute positions, always in ascending
// order and with masked scores contributing exactly zero, so a query's result depends on its position and
// the keys only -- not on how the step was cut, on the batch, or on the pages.
//
// Two kernels share the inner loops:
//  * rows: a CTA owns 64 packed rows (4 warps x 16) of one (request, kv head) and walks all its keys.
//    For portions of prompts.
//  * keys: a request's portion has at most 16 packed rows (a decoded token, or a few); a CTA owns one
//    span of keys, its four warps take 16 keys each of every tile and their running
//    (max, sum, accumulator) are combined in shared memory.  Spans are ranges of absolute positions,
//    whole tiles long; the launcher picks their length so that the CTAs fill the machine in whole
//    waves (att_choose_span); `k_attention_merge` combines them in ascending order.
// K and V rows are gathered page by page with 16-byte cp.async copies (any page size), double buffered.
// With head sizes 64 and 128 and power-of-two pages the keys kernel fetches whole page blocks with bulk copies
// (k_attention_keys_tma: spans, combined inside a cluster where all of them are resident at once;
// k_attention_keys_even: the tiles of all requests cut into one equal run per resident CTA, for many or unequal requests).
#include "common.cuh"
#include <math.h>
#include <cuda.h>

#define ATT_TILE 64            // keys per tile
#define ATT_ROWS 64            // packed query rows per CTA in the rows kernel
#define ATT_KEYS_SLOTS (3 * xr_sm_count())   // CTAs of the keys kernel that are resident at once (two stages: three per SM)
#define ATT_MAX_SPLITS 256     // most spans per request
#define ATT_CLUSTER_MAX 8      // most spans that one cluster combines (the portable cluster size)
#define ATT_THREADS 128

struct AttnMmaArgs {
    const __nv_bfloat16* q;      // token t, head h at q + t * q_stride + h * hd
    __nv_bfloat16* out;          // [n, H * hd]
    const __nv_bfloat16* cache_k;
    const int* seg_start;        // [n_seg] first flat token of the portion
    const int* seg_len;          // [n_seg]
    const int* seg_pos0;         // [n_seg] position of its first token
    const int* block_tables;     // [n_seg][max_pages]
    float* part_acc;             // keys kernel: [n_seg][K][splits][16][hd]
    float* part_ml;              // keys kernel: [n_seg][K][splits][16][2]
    long long q_stride, page_stride, v_offset;
    int H, K, G, max_pages, page_size, window, max_splits;
    int span;                    // keys kernel: keys per span, a multiple of ATT_TILE
    float scale;
    int page_shift;              // log2(page_size) when it is a power of two, else -1
    // bulk-copy (TMA) variant of the keys kernel: the whole cache group as rows of head_dim elements
    int n_layers, layer;         // layers in the cache group, this layer's index
    int* status;                 // set non-zero if a bounded wait gives up
    int recv_rows;               // cluster variant: most packed rows any request of the step has (sizes what a block receives)
};

// Span length (keys) of the keys kernel for a step whose longest request covers `range` keys and that has
// `items` (request, kv head) pairs.  The kernel runs in waves of ATT_KEYS_SLOTS CTAs and a CTA costs about two
// tiles' worth of time before its first keys arrive, so the span that minimises waves x (2 + tiles per span) is
// taken: few requests are cut finely enough to fill the machine, many are cut so that the last wave is full.
// The partition into spans changes only the order of the float32 sums, never which keys a query sees.
static int att_choose_span(int range, long long items) {
    int tiles = (range + ATT_TILE - 1) / ATT_TILE;
    if (tiles < 1) tiles = 1;
    if (items < 1) items = 1;
    // Many requests with short contexts: one span each.  The requests alone fill the machine, a span's tail is short,
    // and a single span writes its output itself, so no merge follows (batch 64 at a context of 704, head size 128:
    // 41 us against 37 + 8 us with four spans and their merge).
    if (items >= ATT_KEYS_SLOTS && tiles <= 16) return tiles * ATT_TILE;
    // Times in nanoseconds, fitted to measurements at head size 128: a wave costs about 4 us before its first
    // keys arrive plus its tiles; a tile streams in 0.9 us when a CTA has an SM to itself (latency bound) and in
    // 2.1 us when the machine is full (bandwidth bound); the merge costs about 0.1 us per span.  (One request of
    // 131,072 keys: 19 spans, a CTA per SM, 100 us; 27 spans, three CTAs on two SMs, 86 us; 55 spans, three per SM, 89 us.)
    int best = tiles;
    long long best_cost = -1;
    for (int s = tiles; s >= 1; s--) {
        int splits = (tiles + s - 1) / s;
        if (splits + 1 > ATT_MAX_SPLITS) break;
        long long ctas = items * splits;
        long long waves = (ctas + ATT_KEYS_SLOTS - 1) / ATT_KEYS_SLOTS;
        long long tile_ns = 2100 * (ctas < ATT_KEYS_SLOTS ? ctas : ATT_KEYS_SLOTS) / ATT_KEYS_SLOTS;
        if (tile_ns < 900) tile_ns = 900;
        long long cost = waves * (4000 + s * tile_ns) + 100LL * splits;
        // spans that are not combined inside clusters (too many, or their blocks would not all be resident: the launcher's
        // rule) are combined by a kernel of its own, which costs that much more than the exchange inside a cluster (4
        // requests at 8,192 keys: 7 spans in clusters 3.62 ms a step, 8 spans and the merge kernel 3.72 ms; but one request
        // at 2,048 keys: 16 spans and the merge kernel 3.07 ms, 8 spans in a cluster 3.13 ms)
        if (splits > ATT_CLUSTER_MAX || ctas + 8LL * (splits - 1) > 2LL * xr_sm_count()) cost += 700;
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = s; }
    }
    return best * ATT_TILE;
}
static int att_range(int max_kv_len, int window) { return window > 0 && window + 16 < max_kv_len ? window + 16 : max_kv_len; }

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Gather one tile of keys AND values [ATT_TILE][HD] each into shared memory rows of HD + 8 elements.
// Rows at positions outside [lo, hi] or on a page the request no longer holds are zero-filled.
// A thread keeps one 16-byte column and walks rows, so the page of a row is looked up once for K and V.
template <int HD>
__device__ __forceinline__ void load_kv_tile(__nv_bfloat16* kdst, __nv_bfloat16* vdst, const AttnMmaArgs& a, const int* bt,
                                             int kvh, int key0, int lo, int hi) {
    constexpr int CH = HD / 8;                       // 16-byte chunks per row
    constexpr int LD = HD + 8;
    constexpr int CT = (CH == 2 || CH == 4 || CH == 8 || CH == 16) ? CH : 1;     // threads across a row
    constexpr int RPP = ATT_THREADS / CT;            // rows per pass
    const int c = threadIdx.x % CT, r0 = threadIdx.x / CT;
    const long long head_off = (long long)kvh * a.page_size * HD;
#pragma unroll 2
    for (int r = r0; r < ATT_TILE; r += RPP) {
        int kp = key0 + r;
        int page = -1, off = 0;
        if (kp >= lo && kp <= hi) {
            int pi;
            if (a.page_shift >= 0) { pi = kp >> a.page_shift; off = kp & (a.page_size - 1); }
            else { pi = kp / a.page_size; off = kp - pi * a.page_size; }
            page = bt[pi];
        }
        __nv_bfloat16* kd = kdst + r * LD;
        __nv_bfloat16* vd = vdst + r * LD;
        if (page >= 0) {
            const __nv_bfloat16* src = a.cache_k + (long long)page * a.page_stride + head_off + (long long)off * HD;
            if (CT == CH) {
                cp_async16(kd + c * 8, src + c * 8);
                cp_async16(vd + c * 8, src + a.v_offset + c * 8);
            } else {
#pragma unroll
                for (int cc = 0; cc < CH; cc++) { cp_async16(kd + cc * 8, src + cc * 8); cp_async16(vd + cc * 8, src + a.v_offset + cc * 8); }
            }
        } else {
            if (CT == CH) {
                *reinterpret_cast<uint4*>(kd + c * 8) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(vd + c * 8) = make_uint4(0, 0, 0, 0);
            } else {
#pragma unroll
                for (int cc = 0; cc < CH; cc++) {
                    *reinterpret_cast<uint4*>(kd + cc * 8) = make_uint4(0, 0, 0, 0);
                    *reinterpret_cast<uint4*>(vd + cc * 8) = make_uint4(0, 0, 0, 0);
                }
            }
        }
    }
}

// One tile of the online softmax for a warp's 16 rows against NKT n-tiles (8 keys each) starting at
// column `col0` of the shared tile:  S = Q K^T, mask, running max/sum, O += P V.
// exp() of the softmax: ex2.approx on a pre-scaled argument (relative error ~2^-22, far below the bfloat16
// rounding of the probabilities that follows)
__device__ __forceinline__ float att_exp(float x) { return __expf(x); }

// LOWER_ONLY: rows 8..15 of the warp's tile hold no query (a decoded token with at most 8 heads per kv head),
// so their softmax and rescaling are skipped (the matrix instruction computes them regardless).
// Element (row, col) of a [64][HD] tile in shared memory.  Plain: rows of HD + 8 elements (the copy kernels'
// layout).  SWZ: what TMA writes with the 128-byte swizzle: sub-tiles of 64 columns, rows of 128 bytes, the
// 16-byte chunk index XORed with the row's low three bits (col must be a multiple of 8).
template <int HD, bool SWZ>
__device__ __forceinline__ const __nv_bfloat16* tile_ptr(const __nv_bfloat16* base, int row, int col) {
    if (SWZ) return base + (col >> 6) * (ATT_TILE * 64) + row * 64 + ((((col & 63) >> 3) ^ (row & 7)) << 3);
    return base + row * (HD + 8) + col;
}

template <int HD, int NKT, bool LOWER_ONLY = false, bool SWZ = false>
__device__ __forceinline__ void tile_step(const uint32_t (*qf)[4], const __nv_bfloat16* ks, const __nv_bfloat16* vs,
                                          int col0, int key0, int pos_a, int pos_b, int window, float scale,
                                          float* m, float* l, float (*o)[4]) {
    const int lane = threadIdx.x & 31;
    float s[NKT][4];
#pragma unroll
    for (int j = 0; j < NKT; j++) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
    for (int kk = 0; kk < HD / 16; kk++) {
#pragma unroll
        for (int j = 0; j < NKT; j += 2) {
            uint32_t b0, b1, b2, b3;
            const __nv_bfloat16* p = tile_ptr<HD, SWZ>(ks, col0 + j * 8 + (lane & 7) + ((lane >> 4) << 3), kk * 16 + (((lane >> 3) & 1) << 3));
            ldsm_x4(b0, b1, b2, b3, p);
            mma_bf16(s[j], qf[kk], b0, b1);
            mma_bf16(s[j + 1], qf[kk], b2, b3);
        }
    }
    // mask and scale: element (row a: c0,c1 ; row b: c2,c3) of n-tile j is key key0 + col0 + 8j + 2t (+1)
    const int t2 = (lane & 3) * 2;
    const int lo_a = window > 0 ? pos_a - window + 1 : 0, lo_b = window > 0 ? pos_b - window + 1 : 0;
    float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
    for (int j = 0; j < NKT; j++) {
#pragma unroll
        for (int e = 0; e < 2; e++) {
            int kp = key0 + col0 + j * 8 + t2 + e;
            float va = (kp <= pos_a && kp >= lo_a) ? s[j][e] * scale : -INFINITY;
            s[j][e] = va;
            mx_a = fmaxf(mx_a, va);
            if (!LOWER_ONLY) {
                float vb = (kp <= pos_b && kp >= lo_b) ? s[j][2 + e] * scale : -INFINITY;
                s[j][2 + e] = vb;
                mx_b = fmaxf(mx_b, vb);
            }
        }
    }
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1)); mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
    if (!LOWER_ONLY) { mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1)); mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2)); }
    float mn_a = fmaxf(m[0], mx_a), mn_b = LOWER_ONLY ? -INFINITY : fmaxf(m[1], mx_b);
    // a row that has seen no key yet keeps max = -inf; subtracting 0 instead keeps exp() at exactly 0
    float off_a = mn_a == -INFINITY ? 0.f : mn_a, off_b = mn_b == -INFINITY ? 0.f : mn_b;
    // the running sums and accumulators are rescaled only when some row's maximum moved
    bool moved = (mn_a != m[0]) || (!LOWER_ONLY && mn_b != m[1]);
    float ca = 1.f, cb = 1.f;
    if (__any_sync(0xffffffffu, moved)) {
        ca = att_exp(m[0] - off_a);                               // m = -inf -> 0
        if (!LOWER_ONLY) cb = att_exp(m[1] - off_b);
#pragma unroll
        for (int d = 0; d < HD / 8; d++) {
            o[d][0] *= ca; o[d][1] *= ca;
            if (!LOWER_ONLY) { o[d][2] *= cb; o[d][3] *= cb; }
        }
    }
    m[0] = mn_a; if (!LOWER_ONLY) m[1] = mn_b;
    float sa = 0.f, sb = 0.f;
#pragma unroll
    for (int j = 0; j < NKT; j++) {
        s[j][0] = att_exp(s[j][0] - off_a); s[j][1] = att_exp(s[j][1] - off_a);
        sa += s[j][0] + s[j][1];
        if (!LOWER_ONLY) {
            s[j][2] = att_exp(s[j][2] - off_b); s[j][3] = att_exp(s[j][3] - off_b);
            sb += s[j][2] + s[j][3];
        } else {
            s[j][2] = 0.f; s[j][3] = 0.f;
        }
    }
    sa += __shfl_xor_sync(0xffffffffu, sa, 1); sa += __shfl_xor_sync(0xffffffffu, sa, 2);
    l[0] = l[0] * ca + sa;
    if (!LOWER_ONLY) {
        sb += __shfl_xor_sync(0xffffffffu, sb, 1); sb += __shfl_xor_sync(0xffffffffu, sb, 2);
        l[1] = l[1] * cb + sb;
    }
    // O += P V, 16 keys per step
#pragma unroll
    for (int kk = 0; kk < NKT / 2; kk++) {
        uint32_t a[4] = {pack_bf16(s[2 * kk][0], s[2 * kk][1]), pack_bf16(s[2 * kk][2], s[2 * kk][3]),
                         pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3])};
#pragma unroll
        for (int d = 0; d < HD / 8; d += 2) {
            uint32_t b0, b1, b2, b3;
            const __nv_bfloat16* p = tile_ptr<HD, SWZ>(vs, col0 + kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), d * 8 + ((lane >> 4) << 3));
            ldsm_x4_t(b0, b1, b2, b3, p);
            mma_bf16(o[d], a, b0, b1);
            mma_bf16(o[d + 1], a, b2, b3);
        }
    }
}

// Q rows of this CTA -> shared [ATT_ROWS or 16][HD + 8]; rows past the portion are zero.
template <int HD>
__device__ __forceinline__ void load_q(__nv_bfloat16* qs, const AttnMmaArgs& a, int tok_base, int kvh, int row0, int rows,
                                       int rows_total) {
    constexpr int CH = HD / 8, LD = HD + 8;
    for (int i = threadIdx.x; i < rows * CH; i += ATT_THREADS) {
        int r = i / CH, c = i % CH;
        int pr = row0 + r;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (pr < rows_total) {
            int tok = tok_base + pr / a.G, head = kvh * a.G + pr % a.G;
            v = *reinterpret_cast<const uint4*>(a.q + (long long)tok * a.q_stride + (long long)head * HD + c * 8);
        }
        *reinterpret_cast<uint4*>(qs + r * LD + c * 8) = v;
    }
}

// ---------------------------------------------------------------------------------------------
// rows kernel: grid (q tiles, K, segments)
// ---------------------------------------------------------------------------------------------
template <int HD>
__global__ void __launch_bounds__(ATT_THREADS)
k_attention_rows(AttnMmaArgs a, int n_seg) {
    xr_pdl_launch();
    constexpr int LD = HD + 8;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __nv_bfloat16* qs = (__nv_bfloat16*)smem_raw;                 // [64][LD]
    __nv_bfloat16* kbuf = qs + ATT_ROWS * LD;                      // [2][64][LD]
    __nv_bfloat16* vbuf = kbuf + 2 * ATT_TILE * LD;                // [2][64][LD]
    // The row tiles of the portions with more than 16 packed rows, laid end to end, are the grid's x (short portions
    // belong to the keys kernel and have no blocks here); a block finds its (portion, tile) by walking the lengths.
    const int kvh = blockIdx.y;
    int seg = -1, tile = 0;
    {
        int before = 0;
        for (int s = 0; s < n_seg; s++) {
            const int rows = a.seg_len[s] * a.G;
            const int t = rows > 16 ? (rows + ATT_ROWS - 1) / ATT_ROWS : 0;
            if ((int)blockIdx.x < before + t) { seg = s; tile = (int)blockIdx.x - before; break; }
            before += t;
        }
    }
    if (seg < 0) return;                                           // (the caller gave an upper bound of the tiles)
    xr_pdl_wait();
    const int L = a.seg_len[seg], rows_total = L * a.G, row0 = tile * ATT_ROWS;
    const int pos0 = a.seg_pos0[seg], tok_base = a.seg_start[seg];
    const int* bt = a.block_tables + (size_t)seg * a.max_pages;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    load_q<HD>(qs, a, tok_base, kvh, row0, ATT_ROWS, rows_total);
    const int last_row = min(rows_total, row0 + ATT_ROWS) - 1;
    const int hi = pos0 + last_row / a.G;                                            // last key any row may read
    const int lo = a.window > 0 ? max(0, pos0 + row0 / a.G - a.window + 1) : 0;       // first key any row may read
    const int t_lo = lo / ATT_TILE, t_hi = hi / ATT_TILE;
    load_kv_tile<HD>(kbuf, vbuf, a, bt, kvh, t_lo * ATT_TILE, lo, hi);
    cp_async_commit();
    __syncthreads();
    uint32_t qf[HD / 16][4];
#pragma unroll
    for (int kk = 0; kk < HD / 16; kk++)
        ldsm_x4(qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], qs + (warp * 16 + (lane & 15)) * LD + kk * 16 + ((lane >> 4) << 3));
    const int ra = row0 + warp * 16 + (lane >> 2), rb = ra + 8;
    const int pos_a = ra < rows_total ? pos0 + ra / a.G : -1, pos_b = rb < rows_total ? pos0 + rb / a.G : -1;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[HD / 8][4];
#pragma unroll
    for (int d = 0; d < HD / 8; d++) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }
    // a warp whose rows all end before a tile starts has nothing to do in it
    const int warp_hi = pos0 + min(last_row, row0 + warp * 16 + 15) / a.G;

    for (int t = t_lo; t <= t_hi; t++) {
        int cur = (t - t_lo) & 1;
        if (t < t_hi) {
            load_kv_tile<HD>(kbuf + (cur ^ 1) * ATT_TILE * LD, vbuf + (cur ^ 1) * ATT_TILE * LD, a, bt, kvh, (t + 1) * ATT_TILE, lo, hi);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (t * ATT_TILE <= warp_hi)
            tile_step<HD, 8>(qf, kbuf + cur * ATT_TILE * LD, vbuf + cur * ATT_TILE * LD, 0, t * ATT_TILE, pos_a, pos_b,
                             a.window, a.scale, m, l, o);
        __syncthreads();
    }
    // rows a (lane/4) and b (+8): columns d*8 + 2*(lane%4) (+1)
    const int t2 = (lane & 3) * 2;
#pragma unroll
    for (int half = 0; half < 2; half++) {
        int pr = half ? rb : ra;
        if (pr >= rows_total) continue;
        float inv = 1.0f / l[half];
        __nv_bfloat16* dst = a.out + ((long long)(tok_base + pr / a.G) * a.H + (kvh * a.G + pr % a.G)) * HD;
#pragma unroll
        for (int d = 0; d < HD / 8; d++)
            *reinterpret_cast<uint32_t*>(dst + d * 8 + t2) = pack_bf16(o[d][2 * half] * inv, o[d][2 * half + 1] * inv);
    }
}

// ---------------------------------------------------------------------------------------------
// keys kernel: grid (spans, K, segments); portions of at most 16 packed rows
// ---------------------------------------------------------------------------------------------
// ATT_KSTAGES: shared-memory stages.  Two let three CTAs share an SM (best when the grid fills the machine
// several times over); four keep one CTA's copies far enough ahead when it has the SM to itself.
template <int HD, int ATT_KSTAGES>
__global__ void __launch_bounds__(ATT_THREADS)
k_attention_keys(AttnMmaArgs a) {
    xr_pdl_launch();
    xr_pdl_wait();
    constexpr int LD = HD + 8;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __nv_bfloat16* qs = (__nv_bfloat16*)smem_raw;                 // [16][LD]
    __nv_bfloat16* kbuf = qs + 16 * LD;                            // [ATT_KSTAGES][64][LD]
    __nv_bfloat16* vbuf = kbuf + ATT_KSTAGES * ATT_TILE * LD;      // [ATT_KSTAGES][64][LD]
    const int seg = blockIdx.z, kvh = blockIdx.y, span = blockIdx.x;
    const int L = a.seg_len[seg], rows_total = L * a.G;
    if (rows_total > 16) return;
    const int pos0 = a.seg_pos0[seg], tok_base = a.seg_start[seg];
    const int hi_all = pos0 + L - 1;
    const int lo_all = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
    const int SPAN = a.span;
    const int first_span = lo_all / SPAN;
    const int k_begin = (first_span + span) * SPAN;                // spans are fixed ranges of absolute positions
    if (k_begin > hi_all) return;
    const int lo = max(lo_all, k_begin), hi = min(hi_all, k_begin + SPAN - 1);
    const int* bt = a.block_tables + (size_t)seg * a.max_pages;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    load_q<HD>(qs, a, tok_base, kvh, 0, 16, rows_total);
    const int t_lo = lo / ATT_TILE, t_hi = hi / ATT_TILE;
    // ring of ATT_KSTAGES tiles: tiles t+1 .. t+ATT_KSTAGES-1 are in flight while tile t is used
#pragma unroll
    for (int i = 0; i < ATT_KSTAGES - 1; i++) {
        if (t_lo + i <= t_hi)
            load_kv_tile<HD>(kbuf + i * ATT_TILE * LD, vbuf + i * ATT_TILE * LD, a, bt, kvh, (t_lo + i) * ATT_TILE, lo, hi);
        cp_async_commit();
    }
    __syncthreads();
    uint32_t qf[HD / 16][4];
#pragma unroll
    for (int kk = 0; kk < HD / 16; kk++)
        ldsm_x4(qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], qs + (lane & 15) * LD + kk * 16 + ((lane >> 4) << 3));
    const int ra = lane >> 2, rb = ra + 8;
    const int pos_a = ra < rows_total ? pos0 + ra / a.G : -1, pos_b = rb < rows_total ? pos0 + rb / a.G : -1;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[HD / 8][4];
#pragma unroll
    for (int d = 0; d < HD / 8; d++) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }

    for (int t = t_lo; t <= t_hi; t++) {
        int cur = (t - t_lo) % ATT_KSTAGES;
        int nxt = (t - t_lo + ATT_KSTAGES - 1) % ATT_KSTAGES;
        if (t + ATT_KSTAGES - 1 <= t_hi)
            load_kv_tile<HD>(kbuf + nxt * ATT_TILE * LD, vbuf + nxt * ATT_TILE * LD, a, bt, kvh, (t + ATT_KSTAGES - 1) * ATT_TILE, lo, hi);
        cp_async_commit();
        cp_async_wait<ATT_KSTAGES - 1>();
        __syncthreads();
        // warp w takes keys [16w, 16w + 16) of the tile; every key of these tiles lies inside the span, and
        // keys outside [lo, hi] are outside every row's own range, so the per-row mask is all that is needed
        int c0 = warp * 16, kfirst = t * ATT_TILE + c0;
        if (kfirst <= hi && kfirst + 15 >= lo) {
            if (rows_total <= 8)
                tile_step<HD, 2, true>(qf, kbuf + cur * ATT_TILE * LD, vbuf + cur * ATT_TILE * LD, c0, t * ATT_TILE, pos_a, pos_b,
                                       a.window, a.scale, m, l, o);
            else
                tile_step<HD, 2, false>(qf, kbuf + cur * ATT_TILE * LD, vbuf + cur * ATT_TILE * LD, c0, t * ATT_TILE, pos_a, pos_b,
                                        a.window, a.scale, m, l, o);
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    // combine the four warps: shared [4][16][HD] accumulators and [4][16][2] (max, sum); the key tiles are done with
    float* acc_s = reinterpret_cast<float*>(kbuf);
    float* ml_s = acc_s + 4 * 16 * HD;
    const int t2 = (lane & 3) * 2;
#pragma unroll
    for (int d = 0; d < HD / 8; d++) {
        acc_s[(warp * 16 + ra) * HD + d * 8 + t2] = o[d][0]; acc_s[(warp * 16 + ra) * HD + d * 8 + t2 + 1] = o[d][1];
        acc_s[(warp * 16 + rb) * HD + d * 8 + t2] = o[d][2]; acc_s[(warp * 16 + rb) * HD + d * 8 + t2 + 1] = o[d][3];
    }
    if ((lane & 3) == 0) {
        ml_s[(warp * 16 + ra) * 2] = m[0]; ml_s[(warp * 16 + ra) * 2 + 1] = l[0];
        ml_s[(warp * 16 + rb) * 2] = m[1]; ml_s[(warp * 16 + rb) * 2 + 1] = l[1];
    }
    __syncthreads();
    size_t item = ((size_t)seg * a.K + kvh) * a.max_splits + span;
    float* pacc = a.part_acc + item * 16 * HD;
    float* pml = a.part_ml + item * 16 * 2;
    for (int i = threadIdx.x; i < rows_total * HD; i += ATT_THREADS) {
        int r = i / HD, d = i % HD;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; w++) mm = fmaxf(mm, ml_s[(w * 16 + r) * 2]);
        float off = mm == -INFINITY ? 0.f : mm;
        float acc = 0.f, ll = 0.f;
#pragma unroll
        for (int w = 0; w < 4; w++) {
            float f = expf(ml_s[(w * 16 + r) * 2] - off);
            acc += acc_s[(w * 16 + r) * HD + d] * f;
            ll += ml_s[(w * 16 + r) * 2 + 1] * f;
        }
        pacc[r * HD + d] = acc;
        if (d == 0) { pml[r * 2] = mm; pml[r * 2 + 1] = ll; }
    }
}

// ---------------------------------------------------------------------------------------------
// keys kernel with bulk copies: same work split and arithmetic as k_attention_keys, but one thread fetches
// each tile with TMA (cp.async.bulk.tensor, 128-byte swizzle) straight from the pages: the cache group is
// one 2-D tensor [(page, layer, K|V, kv head, token)][head_dim], a page's block of one kv head is
// min(page_size, 64) consecutive rows.  No thread computes gather addresses.  Needs head_dim 64 or 128 and a
// power-of-two page size >= 8.  Rows beyond a request's last key are not zero-filled by the copy; scores there
// are masked, and the value rows are cleared in shared memory so that stale bytes cannot reach the output.
// ---------------------------------------------------------------------------------------------
#define ATT_SPIN_LIMIT (1u << 22)

__device__ __forceinline__ uint32_t att_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool att_mbar_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < ATT_SPIN_LIMIT; i++) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(att_smem_u32(bar)), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

// CLUSTER: the spans of one (request, kv head) are the blocks of one thread-block cluster (grid.x = cluster size <=
// 8) and combine their results among themselves: every block sends each block the slice of its accumulator that
// block is to finish, and its rows' (maximum, sum) pairs, into that block's shared memory; after one cluster barrier
// each block weighs and adds what it received, in ascending span order, and writes its slice of the output rows.
// The partial results then never leave the SMs and no merge kernel follows.
__device__ __forceinline__ uint32_t att_map_to_rank(const void* mine, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(att_smem_u32(mine)), "r"(rank));
    return remote;
}
__device__ __forceinline__ void att_cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void att_cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

template <int HD, int STAGES, bool CLUSTER>
__global__ void __launch_bounds__(ATT_THREADS)
k_attention_keys_tma(const __grid_constant__ CUtensorMap cache_map, AttnMmaArgs a) {
    xr_pdl_launch();
    constexpr int LD = HD + 8;
    constexpr int QUADS = HD / 4;
    constexpr int TILE_ELEMS = ATT_TILE * HD;                      // one K (or V) tile, swizzled sub-tiles of 64 columns
    extern __shared__ __align__(16) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);     // TMA with the 128-byte swizzle wants 1 KB
    __nv_bfloat16* kbuf = (__nv_bfloat16*)smem;                    // [STAGES][TILE_ELEMS]
    __nv_bfloat16* vbuf = kbuf + STAGES * TILE_ELEMS;              // [STAGES][TILE_ELEMS]
    __nv_bfloat16* qs = vbuf + STAGES * TILE_ELEMS;                // [16][LD]
    uint64_t* full = (uint64_t*)(qs + 16 * LD);
    volatile int* gave_up = (volatile int*)(full + STAGES);
    // CLUSTER: what the other spans send.  Nothing else lives here: a span that is done early writes into the
    // shared memory of one that is still at work.
    float4* recv_acc = (float4*)(((uintptr_t)(gave_up + 1) + 15) & ~(uintptr_t)15);      // [spans][per] quadruples
    float2* recv_ml = (float2*)(recv_acc + a.recv_rows * QUADS + ATT_CLUSTER_MAX);       // [spans][16] (maximum, sum)
    const int seg = blockIdx.z, kvh = blockIdx.y, span = blockIdx.x;
    const int L = a.seg_len[seg], rows_total = L * a.G;
    if (rows_total > 16) return;                                   // (the whole cluster: it shares the request)
    const int pos0 = a.seg_pos0[seg], tok_base = a.seg_start[seg];
    const int hi_all = pos0 + L - 1;
    const int lo_all = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
    const int SPAN = a.span;
    const int first_span = lo_all / SPAN;
    const int k_begin = (first_span + span) * SPAN;
    const int n_spans = hi_all / SPAN - first_span + 1;            // spans of this request that hold keys
    if (CLUSTER) att_cluster_arrive();                             // "this block runs": waited for before anyone writes to it
    if (k_begin > hi_all) {
        // no keys for this span: nobody sends to it and it owns no output, but the cluster's barriers count it
        if (CLUSTER) { att_cluster_wait(); att_cluster_arrive(); att_cluster_wait(); }
        return;
    }
    const int lo = max(lo_all, k_begin), hi = min(hi_all, k_begin + SPAN - 1);
    const int* bt = a.block_tables + (size_t)seg * a.max_pages;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t_lo = lo / ATT_TILE, t_hi = hi / ATT_TILE;
    const int box_rows = a.page_size < ATT_TILE ? a.page_size : ATT_TILE;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(att_smem_u32(&full[s])), "r"(1));
        *gave_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // one thread fetches tile `t` into stage `s`: K and V, per page block and per 64-column half
    auto fetch = [&](int t, int s) {
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(att_smem_u32(&full[s])), "r"(2 * TILE_ELEMS * 2) : "memory");
        for (int r0 = 0; r0 < ATT_TILE; r0 += box_rows) {
            int kp = t * ATT_TILE + r0;
            const int pi = kp >> a.page_shift;
            int page = pi < a.max_pages ? bt[pi] : -1;             // -1 (no page): the copy reads outside the tensor and fills zeros
            int tok = kp & (a.page_size - 1);
            long long rowk = ((((long long)page * a.n_layers + a.layer) * 2 + 0) * a.K + kvh) * a.page_size + tok;
            long long rowv = rowk + (long long)a.K * a.page_size;
            if (page < 0) { rowk = -(long long)ATT_TILE; rowv = -(long long)ATT_TILE; }
#pragma unroll
            for (int c = 0; c < HD / 64; c++) {
                __nv_bfloat16* kd = kbuf + s * TILE_ELEMS + c * (ATT_TILE * 64) + r0 * 64;
                __nv_bfloat16* vd = vbuf + s * TILE_ELEMS + c * (ATT_TILE * 64) + r0 * 64;
                asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                             ::"r"(att_smem_u32(kd)), "l"(&cache_map), "r"(c * 64), "r"((int)rowk), "r"(att_smem_u32(&full[s])) : "memory");
                asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                             ::"r"(att_smem_u32(vd)), "l"(&cache_map), "r"(c * 64), "r"((int)rowv), "r"(att_smem_u32(&full[s])) : "memory");
            }
        }
    };
    // The step's description and the keys of earlier steps do not change while the step runs: a span that ends
    // before the step's own tokens starts its copies before the kernel ahead in the stream is complete.
    const bool old_keys_only = hi < pos0;
    if (threadIdx.x == 0 && old_keys_only)
        for (int i = 0; i < STAGES - 1 && t_lo + i <= t_hi; i++) fetch(t_lo + i, i);
    xr_pdl_wait();
    if (threadIdx.x == 0 && !old_keys_only)
        for (int i = 0; i < STAGES - 1 && t_lo + i <= t_hi; i++) fetch(t_lo + i, i);
    load_q<HD>(qs, a, tok_base, kvh, 0, 16, rows_total);
    __syncthreads();
    uint32_t qf[HD / 16][4];
#pragma unroll
    for (int kk = 0; kk < HD / 16; kk++)
        ldsm_x4(qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], qs + (lane & 15) * LD + kk * 16 + ((lane >> 4) << 3));
    const int ra = lane >> 2, rb = ra + 8;
    const int pos_a = ra < rows_total ? pos0 + ra / a.G : -1, pos_b = rb < rows_total ? pos0 + rb / a.G : -1;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[HD / 8][4];
#pragma unroll
    for (int d = 0; d < HD / 8; d++) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }

    for (int t = t_lo; t <= t_hi; t++) {
        int i = t - t_lo, cur = i % STAGES;
        if (threadIdx.x == 0 && t + STAGES - 1 <= t_hi) fetch(t + STAGES - 1, (i + STAGES - 1) % STAGES);
        // A wait that runs out does not leave the loop (the threads of a CTA must keep meeting at the barriers
        // below); it is recorded, the result of this CTA is then meaningless, and the status word says so.
        if (!att_mbar_wait(&full[cur], (i / STAGES) & 1)) *gave_up = 1;
        __nv_bfloat16* vt = vbuf + cur * TILE_ELEMS;
        if ((t + 1) * ATT_TILE - 1 > hi) {
            // the tile runs past the last key: clear those value rows (probabilities there are zero, but 0 x garbage
            // must stay 0 whatever the bytes are)
            int first_bad = hi + 1 - t * ATT_TILE;
            for (int e = threadIdx.x; e < (ATT_TILE - first_bad) * (HD / 8); e += ATT_THREADS) {
                int r = first_bad + e / (HD / 8), c = (e % (HD / 8)) * 8;
                *reinterpret_cast<uint4*>(const_cast<__nv_bfloat16*>(tile_ptr<HD, true>(vt, r, c))) = make_uint4(0, 0, 0, 0);
            }
            __syncthreads();
        }
        if (t * ATT_TILE < lo) {
            int n_bad = lo - t * ATT_TILE;
            for (int e = threadIdx.x; e < n_bad * (HD / 8); e += ATT_THREADS) {
                int r = e / (HD / 8), c = (e % (HD / 8)) * 8;
                *reinterpret_cast<uint4*>(const_cast<__nv_bfloat16*>(tile_ptr<HD, true>(vt, r, c))) = make_uint4(0, 0, 0, 0);
            }
            __syncthreads();
        }
        int c0 = warp * 16, kfirst = t * ATT_TILE + c0;
        if (kfirst <= hi && kfirst + 15 >= lo) {
            if (rows_total <= 8)
                tile_step<HD, 2, true, true>(qf, kbuf + cur * TILE_ELEMS, vt, c0, t * ATT_TILE, pos_a, pos_b, a.window, a.scale, m, l, o);
            else
                tile_step<HD, 2, false, true>(qf, kbuf + cur * TILE_ELEMS, vt, c0, t * ATT_TILE, pos_a, pos_b, a.window, a.scale, m, l, o);
        }
        __syncthreads();                 // everyone is done with stage `cur` before it is fetched into again
    }
    __syncthreads();
    if (threadIdx.x == 0 && *gave_up) atomicExch(a.status, 2);
    // combine the four warps (same as the copy kernel); the stage buffers are free now
    float* acc_s = reinterpret_cast<float*>(kbuf);
    float* ml_s = acc_s + 4 * 16 * HD;
    const int t2 = (lane & 3) * 2;
#pragma unroll
    for (int d = 0; d < HD / 8; d++) {
        acc_s[(warp * 16 + ra) * HD + d * 8 + t2] = o[d][0]; acc_s[(warp * 16 + ra) * HD + d * 8 + t2 + 1] = o[d][1];
        acc_s[(warp * 16 + rb) * HD + d * 8 + t2] = o[d][2]; acc_s[(warp * 16 + rb) * HD + d * 8 + t2 + 1] = o[d][3];
    }
    if ((lane & 3) == 0) {
        ml_s[(warp * 16 + ra) * 2] = m[0]; ml_s[(warp * 16 + ra) * 2 + 1] = l[0];
        ml_s[(warp * 16 + rb) * 2] = m[1]; ml_s[(warp * 16 + rb) * 2 + 1] = l[1];
    }
    __syncthreads();
    if (!CLUSTER) {
        size_t item = ((size_t)seg * a.K + kvh) * a.max_splits + span;
        float* pacc = a.part_acc + item * 16 * HD;
        float* pml = a.part_ml + item * 16 * 2;
        for (int i = threadIdx.x; i < rows_total * HD; i += ATT_THREADS) {
            int r = i / HD, d = i % HD;
            float mm = -INFINITY;
#pragma unroll
            for (int w = 0; w < 4; w++) mm = fmaxf(mm, ml_s[(w * 16 + r) * 2]);
            float off = mm == -INFINITY ? 0.f : mm;
            float acc = 0.f, ll = 0.f;
#pragma unroll
            for (int w = 0; w < 4; w++) {
                float f = expf(ml_s[(w * 16 + r) * 2] - off);
                acc += acc_s[(w * 16 + r) * HD + d] * f;
                ll += ml_s[(w * 16 + r) * 2 + 1] * f;
            }
            pacc[r * HD + d] = acc;
            if (d == 0) { pml[r * 2] = mm; pml[r * 2 + 1] = ll; }
        }
        return;
    }
    // Quadruple q of the output rows (row q / QUADS, columns 4 (q % QUADS) ..) is finished by span q % n_spans, which
    // keeps it at [sender][q / n_spans].
    const int owned = rows_total * QUADS, per = (owned + n_spans - 1) / n_spans;
    att_cluster_wait();                                           // every block of the cluster has begun
    if (n_spans == 1) {
        // nothing to exchange: the four warps' sums are the result
        for (int q = threadIdx.x; q < owned; q += ATT_THREADS) {
            const int r = q / QUADS, d = (q % QUADS) * 4;
            float mm = -INFINITY;
#pragma unroll
            for (int w = 0; w < 4; w++) mm = fmaxf(mm, ml_s[(w * 16 + r) * 2]);
            const float off = mm == -INFINITY ? 0.f : mm;
            float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
            float ll = 0.f;
#pragma unroll
            for (int w = 0; w < 4; w++) {
                const float f = expf(ml_s[(w * 16 + r) * 2] - off);
                const float4 v = *reinterpret_cast<const float4*>(acc_s + (w * 16 + r) * HD + d);
                t.x += v.x * f; t.y += v.y * f; t.z += v.z * f; t.w += v.w * f;
                ll += ml_s[(w * 16 + r) * 2 + 1] * f;
            }
            const float inv = 1.0f / ll;
            __nv_bfloat16* dst = a.out + ((long long)(tok_base + r / a.G) * a.H + (kvh * a.G + r % a.G)) * HD + d;
            __nv_bfloat162 lo2 = __floats2bfloat162_rn(t.x * inv, t.y * inv), hi2 = __floats2bfloat162_rn(t.z * inv, t.w * inv);
            uint2 packed;
            packed.x = *reinterpret_cast<uint32_t*>(&lo2);
            packed.y = *reinterpret_cast<uint32_t*>(&hi2);
            *reinterpret_cast<uint2*>(dst) = packed;
        }
        att_cluster_arrive();
        att_cluster_wait();
        return;
    }
    for (int q = threadIdx.x; q < owned; q += ATT_THREADS) {
        const int r = q / QUADS, d = (q % QUADS) * 4;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; w++) mm = fmaxf(mm, ml_s[(w * 16 + r) * 2]);
        const float off = mm == -INFINITY ? 0.f : mm;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        float ll = 0.f;
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const float f = expf(ml_s[(w * 16 + r) * 2] - off);
            const float4 v = *reinterpret_cast<const float4*>(acc_s + (w * 16 + r) * HD + d);
            acc.x += v.x * f; acc.y += v.y * f; acc.z += v.z * f; acc.w += v.w * f;
            ll += ml_s[(w * 16 + r) * 2 + 1] * f;
        }
        uint32_t dst = att_map_to_rank(recv_acc + span * per + q / n_spans, (uint32_t)(q % n_spans));
        asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "f"(acc.x), "f"(acc.y), "f"(acc.z), "f"(acc.w) : "memory");
        if (d == 0) {
            for (int o = 0; o < n_spans; o++) {
                uint32_t dm = att_map_to_rank(recv_ml + span * 16 + r, (uint32_t)o);
                asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(dm), "f"(mm), "f"(ll) : "memory");
            }
        }
    }
    att_cluster_arrive();
    att_cluster_wait();
    for (int j = threadIdx.x; j < per; j += ATT_THREADS) {
        const int q = j * n_spans + span;
        if (q >= owned) break;
        const int r = q / QUADS, d = (q % QUADS) * 4;
        float mm = -INFINITY;
        for (int sp = 0; sp < n_spans; sp++) mm = fmaxf(mm, recv_ml[sp * 16 + r].x);
        const float off = mm == -INFINITY ? 0.f : mm;
        float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
        float ll = 0.f;
        for (int sp = 0; sp < n_spans; sp++) {
            const float2 ml = recv_ml[sp * 16 + r];
            const float wk = __expf(ml.x - off);
            const float4 v = recv_acc[sp * per + j];
            t.x += v.x * wk; t.y += v.y * wk; t.z += v.z * wk; t.w += v.w * wk;
            ll += ml.y * wk;
        }
        const float inv = 1.0f / ll;
        __nv_bfloat16* dst = a.out + ((long long)(tok_base + r / a.G) * a.H + (kvh * a.G + r % a.G)) * HD + d;
        __nv_bfloat162 lo2 = __floats2bfloat162_rn(t.x * inv, t.y * inv), hi2 = __floats2bfloat162_rn(t.z * inv, t.w * inv);
        uint2 packed;
        packed.x = *reinterpret_cast<uint32_t*>(&lo2);
        packed.y = *reinterpret_cast<uint32_t*>(&hi2);
        *reinterpret_cast<uint2*>(dst) = packed;
    }
}

// ---------------------------------------------------------------------------------------------
// keys kernel in even shares.  With more (request, kv head) pairs than CTAs fit on the machine, one CTA per pair (or
// per span) runs in waves whose last is mostly idle, and requests of unequal length make it worse.  Here the grid is
// the number of CTAs that are resident at once, and the tiles of all pairs, laid end to end (request, kv head, tile),
// are cut into that many equal runs.  A CTA walks its run with one ring of bulk copies that runs on across the
// pairs it touches.  A pair that lies inside one run is finished there.  A pair that is cut belongs to the CTA that
// holds its first tiles, and that piece is the last of its CTA's run.  Every later piece is the first of its CTA's
// run: that CTA leaves (accumulator, maximum, sum) in its own slot of the scratch and raises its flag; the owner,
// at the very end of its run, takes the pieces in ascending order, lowers the flags again and writes the rows.
// A CTA waits only for CTAs that were given the piece as their first work and wait for nobody before it, and all CTAs
// are resident at once (the grid is sized by the occupancy the runtime reports), so the wait ends; it is bounded all
// the same.  The result is a fixed function of the step's lengths: the same sums in the same order.
// Flags are touched after griddepcontrol.wait only: the launch of the layer before has completed by then.
// ---------------------------------------------------------------------------------------------
#define ATT_EVEN_MAX_SEGS 512

__device__ __forceinline__ int att_ld_acquire(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void att_st_release(int* p, int v) {
    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Wait until the word at `flag` is not zero, at most `limit` looks (each a load from L2).  False: it stayed zero.
__device__ __forceinline__ bool att_wait_flag(const int* flag, uint32_t limit) {
    for (uint32_t spin = 0; spin < limit; spin++)
        if (att_ld_acquire(flag) != 0) return true;
    return false;
}

// The wait of the kernel below on a flag that nothing raises: it runs out after `limit` looks, and the kernel reports it
// in the status word exactly as the attention kernel does.  For tests of what the host does with that word; the
// context stays usable.
__global__ void k_attention_wait_probe(const int* flag, int* status, uint32_t limit) {
    if (!att_wait_flag(flag, limit)) atomicExch(status, 2);
}
XR_EXPORT int xr_attention_wait_probe(const int* flag, int* status, unsigned int limit, cudaStream_t stream) {
    if (flag == nullptr || status == nullptr || limit < 1 || limit > ATT_SPIN_LIMIT) return XR_ERR_ARG;
    k_attention_wait_probe<<<1, 1, 0, stream>>>(flag, status, limit);
    return xr_launch_status();
}

template <int HD, int STAGES>
__global__ void __launch_bounds__(ATT_THREADS, 3)
k_attention_keys_even(const __grid_constant__ CUtensorMap cache_map, AttnMmaArgs a, int n_seg, int* flags) {
    xr_pdl_launch();
    constexpr int LD = HD + 8, QUADS = HD / 4, TILE_ELEMS = ATT_TILE * HD;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if ((att_smem_u32(smem_raw) & 1023u) != 0) {                   // the copies' 128-byte swizzle counts from 1 KB boundaries
        if (tid == 0) atomicExch(a.status, 2);
        return;
    }
    const int R = a.recv_rows;                                     // most packed rows of any request of the step
    __nv_bfloat16* kbuf = (__nv_bfloat16*)smem_raw;                // [STAGES][TILE_ELEMS]
    __nv_bfloat16* vbuf = kbuf + STAGES * TILE_ELEMS;              // [STAGES][TILE_ELEMS]
    uint8_t* rest = (uint8_t*)(vbuf + STAGES * TILE_ELEMS);
    // the Q rows at the start of a piece and the four warps' sums at its end share one region
    __nv_bfloat16* qs = (__nv_bfloat16*)rest;                      // [16][LD]
    float* acc_s = (float*)rest;                                   // [4][R][HD]
    const int shared_region = 16 * LD * 2 > 4 * R * HD * 4 ? 16 * LD * 2 : 4 * R * HD * 4;
    float* ml_s = (float*)(rest + shared_region);                  // [4][16][2]
    uint64_t* full = (uint64_t*)(ml_s + 4 * 16 * 2);
    int* seg_pre = (int*)(full + STAGES);                          // [n_seg + 1]: tiles of the requests before this one
    volatile int* gave_up = (volatile int*)(seg_pre + n_seg + 1);

    // tiles of every request (the step's description does not change while the step runs)
    for (int s = tid; s < n_seg; s += ATT_THREADS) {
        const int L = a.seg_len[s], p0 = a.seg_pos0[s];
        int cnt = 0;
        if (L > 0 && L * a.G <= 16) {
            const int lo = a.window > 0 ? max(0, p0 - a.window + 1) : 0;
            cnt = (p0 + L - 1) / ATT_TILE - lo / ATT_TILE + 1;
        }
        seg_pre[s + 1] = cnt;
    }
    if (tid == 0) {
        seg_pre[0] = 0;
        for (int s = 0; s < STAGES; s++)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(att_smem_u32(&full[s])), "r"(1));
        *gave_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp == 0) {
        int run = 0;
        for (int base = 0; base < n_seg; base += 32) {
            const int s = base + lane;
            int v = s < n_seg ? seg_pre[s + 1] : 0;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int u = __shfl_up_sync(0xffffffffu, v, o);
                if (lane >= o) v += u;
            }
            if (s < n_seg) seg_pre[s + 1] = run + v;
            run += __shfl_sync(0xffffffffu, v, 31);
        }
    }
    __syncthreads();
    const long long T = (long long)a.K * seg_pre[n_seg];
    const long long C = gridDim.x, c = blockIdx.x;
    const long long begin = T * c / C, end = T * (c + 1) / C;
    if (begin >= end) return;
    const int n_mine = (int)(end - begin);

    // the pair and the tile at place f of the row of all tiles; t_first and cnt: the pair's first tile and its tiles
    auto locate = [&](long long f, int& seg, int& kvh, int& t, int& t_first, int& cnt) {
        int lo = 0, hi = n_seg;                                    // K * seg_pre[lo] <= f < K * seg_pre[hi]
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if ((long long)a.K * seg_pre[mid] <= f) lo = mid; else hi = mid;
        }
        seg = lo;
        cnt = seg_pre[lo + 1] - seg_pre[lo];
        const int rem = (int)(f - (long long)a.K * seg_pre[lo]);
        kvh = rem / cnt;
        const int p0 = a.seg_pos0[lo];
        t_first = (a.window > 0 ? max(0, p0 - a.window + 1) : 0) / ATT_TILE;
        t = t_first + rem % cnt;
    };

    // thread 0 keeps the place of the next tile to fetch; tile number i of the run goes to stage i % STAGES
    const int box_rows = a.page_size < ATT_TILE ? a.page_size : ATT_TILE;
    int fs = 0, fk = 0, ft = 0, ft_first = 0, fcnt = 1, fetched = 0;
    if (tid == 0) locate(begin, fs, fk, ft, ft_first, fcnt);
    auto fetch_next = [&]() {
        const int s = fetched % STAGES;
        const int* bt = a.block_tables + (size_t)fs * a.max_pages;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the stage was read, and perhaps partly cleared, by threads
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(att_smem_u32(&full[s])), "r"(2 * TILE_ELEMS * 2) : "memory");
        for (int r0 = 0; r0 < ATT_TILE; r0 += box_rows) {
            const int kp = ft * ATT_TILE + r0;
            const int pi = kp >> a.page_shift;
            const int page = pi < a.max_pages ? bt[pi] : -1;       // -1 (no page): the copy reads outside the tensor and fills zeros
            const int tok = kp & (a.page_size - 1);
            long long rowk = ((((long long)page * a.n_layers + a.layer) * 2 + 0) * a.K + fk) * a.page_size + tok;
            long long rowv = rowk + (long long)a.K * a.page_size;
            if (page < 0) { rowk = -(long long)ATT_TILE; rowv = -(long long)ATT_TILE; }
#pragma unroll
            for (int cc = 0; cc < HD / 64; cc++) {
                __nv_bfloat16* kd = kbuf + s * TILE_ELEMS + cc * (ATT_TILE * 64) + r0 * 64;
                __nv_bfloat16* vd = vbuf + s * TILE_ELEMS + cc * (ATT_TILE * 64) + r0 * 64;
                asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                             ::"r"(att_smem_u32(kd)), "l"(&cache_map), "r"(cc * 64), "r"((int)rowk), "r"(att_smem_u32(&full[s])) : "memory");
                asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                             ::"r"(att_smem_u32(vd)), "l"(&cache_map), "r"(cc * 64), "r"((int)rowv), "r"(att_smem_u32(&full[s])) : "memory");
            }
        }
        fetched++;
        if (++ft == ft_first + fcnt) {                             // on to the next pair
            if (++fk == a.K) {
                fk = 0;
                do { fs++; } while (fs < n_seg && seg_pre[fs + 1] == seg_pre[fs]);
                if (fs < n_seg) {
                    const int p0 = a.seg_pos0[fs];
                    fcnt = seg_pre[fs + 1] - seg_pre[fs];
                    ft_first = (a.window > 0 ? max(0, p0 - a.window + 1) : 0) / ATT_TILE;
                }
            }
            ft = ft_first;
        }
    };
    // tiles that hold keys of earlier steps only may be asked for before the kernel ahead in the stream is complete
    if (tid == 0)
        while (fetched < STAGES && fetched < n_mine && (ft + 1) * ATT_TILE <= a.seg_pos0[fs]) fetch_next();
    xr_pdl_wait();
    if (tid == 0)
        while (fetched < STAGES && fetched < n_mine) fetch_next();
    const int ra = lane >> 2, rb = ra + 8, t2 = (lane & 3) * 2;
    long long pos = begin;
    int i0 = 0;                                                    // number in the run of the piece's first tile
    while (pos < end) {
        int seg, kvh, t_from, t_first, cnt;
        locate(pos, seg, kvh, t_from, t_first, cnt);
        const int L = a.seg_len[seg], rows_total = L * a.G, pos0 = a.seg_pos0[seg], tok_base = a.seg_start[seg];
        const int hi = pos0 + L - 1, lo = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
        const int t_last = t_first + cnt - 1;
        const long long left = end - pos;
        const int n_here = (long long)(t_last - t_from + 1) < left ? t_last - t_from + 1 : (int)left;
        const int t_to = t_from + n_here - 1;
        __syncthreads();                                           // the sums of the piece before have been read
        load_q<HD>(qs, a, tok_base, kvh, 0, 16, rows_total);
        __syncthreads();
        uint32_t qf[HD / 16][4];
#pragma unroll
        for (int kk = 0; kk < HD / 16; kk++)
            ldsm_x4(qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], qs + (lane & 15) * LD + kk * 16 + ((lane >> 4) << 3));
        __syncthreads();                                           // every warp has its Q rows in registers: the region is free for the sums
        const int pos_a = ra < rows_total ? pos0 + ra / a.G : -1, pos_b = rb < rows_total ? pos0 + rb / a.G : -1;
        float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
        float o[HD / 8][4];
#pragma unroll
        for (int d = 0; d < HD / 8; d++) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }

        for (int t = t_from; t <= t_to; t++) {
            const int i = i0 + (t - t_from), cur = i % STAGES;
            if (!att_mbar_wait(&full[cur], (i / STAGES) & 1)) *gave_up = 1;
            __nv_bfloat16* vt = vbuf + cur * TILE_ELEMS;
            if ((t + 1) * ATT_TILE - 1 > hi) {
                // the tile runs past the last key: clear those value rows (0 x garbage must stay 0)
                const int first_bad = hi + 1 - t * ATT_TILE;
                for (int e = tid; e < (ATT_TILE - first_bad) * (HD / 8); e += ATT_THREADS) {
                    const int r = first_bad + e / (HD / 8), cc = (e % (HD / 8)) * 8;
                    *reinterpret_cast<uint4*>(const_cast<__nv_bfloat16*>(tile_ptr<HD, true>(vt, r, cc))) = make_uint4(0, 0, 0, 0);
                }
                __syncthreads();
            }
            if (t * ATT_TILE < lo) {
                const int n_bad = lo - t * ATT_TILE;
                for (int e = tid; e < n_bad * (HD / 8); e += ATT_THREADS) {
                    const int r = e / (HD / 8), cc = (e % (HD / 8)) * 8;
                    *reinterpret_cast<uint4*>(const_cast<__nv_bfloat16*>(tile_ptr<HD, true>(vt, r, cc))) = make_uint4(0, 0, 0, 0);
                }
                __syncthreads();
            }
            const int c0 = warp * 16, kfirst = t * ATT_TILE + c0;
            if (kfirst <= hi && kfirst + 15 >= lo) {
                if (rows_total <= 8)
                    tile_step<HD, 2, true, true>(qf, kbuf + cur * TILE_ELEMS, vt, c0, t * ATT_TILE, pos_a, pos_b, a.window, a.scale, m, l, o);
                else
                    tile_step<HD, 2, false, true>(qf, kbuf + cur * TILE_ELEMS, vt, c0, t * ATT_TILE, pos_a, pos_b, a.window, a.scale, m, l, o);
            }
            __syncthreads();                                       // everyone is done with stage `cur`:
            if (tid == 0 && fetched < n_mine) fetch_next();        // tile i + STAGES goes into it at once, so the ring stays full
        }
        // the four warps' sums side by side
#pragma unroll
        for (int d = 0; d < HD / 8; d++) {
            if (ra < rows_total) { acc_s[(warp * R + ra) * HD + d * 8 + t2] = o[d][0]; acc_s[(warp * R + ra) * HD + d * 8 + t2 + 1] = o[d][1]; }
            if (rb < rows_total) { acc_s[(warp * R + rb) * HD + d * 8 + t2] = o[d][2]; acc_s[(warp * R + rb) * HD + d * 8 + t2 + 1] = o[d][3]; }
        }
        if ((lane & 3) == 0) {
            ml_s[(warp * 16 + ra) * 2] = m[0]; ml_s[(warp * 16 + ra) * 2 + 1] = l[0];
            ml_s[(warp * 16 + rb) * 2] = m[1]; ml_s[(warp * 16 + rb) * 2 + 1] = l[1];
        }
        __syncthreads();
        // this thread's quadruples of the piece's rows: q = tid + ATT_THREADS j is row q / QUADS, columns 4 (q % QUADS) ..
        const int owned = rows_total * QUADS;
        float4 acc[4];
        float mm[4], ll[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int q = tid + j * ATT_THREADS;
            acc[j] = make_float4(0.f, 0.f, 0.f, 0.f); mm[j] = -INFINITY; ll[j] = 0.f;
            if (q < owned) {
                const int r = q / QUADS, d = (q % QUADS) * 4;
#pragma unroll
                for (int w = 0; w < 4; w++) mm[j] = fmaxf(mm[j], ml_s[(w * 16 + r) * 2]);
                const float off = mm[j] == -INFINITY ? 0.f : mm[j];
#pragma unroll
                for (int w = 0; w < 4; w++) {
                    const float f = expf(ml_s[(w * 16 + r) * 2] - off);
                    const float4 v = *reinterpret_cast<const float4*>(acc_s + (w * R + r) * HD + d);
                    acc[j].x += v.x * f; acc[j].y += v.y * f; acc[j].z += v.z * f; acc[j].w += v.w * f;
                    ll[j] += ml_s[(w * 16 + r) * 2 + 1] * f;
                }
            }
        }
        if (t_from != t_first) {
            // a later piece of a pair that began in a CTA before this one: leave it in this CTA's slot
            float* pacc = a.part_acc + (size_t)c * 16 * HD;
            float* pml = a.part_ml + (size_t)c * 32;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int q = tid + j * ATT_THREADS;
                if (q < owned) {
                    const int r = q / QUADS, d = (q % QUADS) * 4;
                    *reinterpret_cast<float4*>(pacc + r * HD + d) = acc[j];
                    if (d == 0) *reinterpret_cast<float2*>(pml + r * 2) = make_float2(mm[j], ll[j]);
                }
            }
            __syncthreads();
            if (tid == 0) { __threadfence(); att_st_release(flags + c, 1); }
        } else {
            if (t_to != t_last) {
                // the first piece of a pair that goes on in the CTAs after this one: theirs, in ascending order
                const long long pair_end = pos + cnt;
                // the CTAs after this one whose runs begin inside the pair (with fewer tiles than CTAs some of them are empty)
                int nf = 0;
                for (long long c2 = c + 1; c2 < C && T * c2 / C < pair_end; c2++) nf++;
                // their flags, each by a thread of its own; a CTA without tiles has nothing to say
                for (int k = tid; k < nf; k += ATT_THREADS) {
                    const long long c2 = c + 1 + k;
                    if (T * c2 / C == T * (c2 + 1) / C) continue;
                    if (att_wait_flag(flags + c2, ATT_SPIN_LIMIT)) *(volatile int*)(flags + c2) = 0; else *gave_up = 1;
                }
                __syncthreads();
                if (!*gave_up) {
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const int q = tid + j * ATT_THREADS;
                        if (q >= owned) continue;
                        const int r = q / QUADS, d = (q % QUADS) * 4;
                        // the piece after the one being added is on its way meanwhile
                        float2 ml_next = make_float2(-INFINITY, 0.f);
                        float4 v_next = make_float4(0.f, 0.f, 0.f, 0.f);
                        auto ask = [&](int k) {
                            const long long c2 = c + 1 + k;
                            if (T * c2 / C == T * (c2 + 1) / C) { ml_next = make_float2(-INFINITY, 0.f); v_next = make_float4(0.f, 0.f, 0.f, 0.f); return; }
                            ml_next = __ldcg(reinterpret_cast<const float2*>(a.part_ml + (size_t)c2 * 32 + r * 2));
                            v_next = __ldcg(reinterpret_cast<const float4*>(a.part_acc + (size_t)c2 * 16 * HD + r * HD + d));
                        };
                        ask(0);
                        for (int k = 0; k < nf; k++) {
                            const float2 ml2 = ml_next;
                            const float4 v = v_next;
                            if (k + 1 < nf) ask(k + 1);
                            const float top = fmaxf(mm[j], ml2.x), off = top == -INFINITY ? 0.f : top;
                            const float f1 = expf(mm[j] - off), f2 = expf(ml2.x - off);
                            acc[j].x = acc[j].x * f1 + v.x * f2; acc[j].y = acc[j].y * f1 + v.y * f2;
                            acc[j].z = acc[j].z * f1 + v.z * f2; acc[j].w = acc[j].w * f1 + v.w * f2;
                            ll[j] = ll[j] * f1 + ml2.y * f2;
                            mm[j] = top;
                        }
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int q = tid + j * ATT_THREADS;
                if (q < owned) {
                    const int r = q / QUADS, d = (q % QUADS) * 4;
                    const float inv = 1.0f / ll[j];
                    __nv_bfloat16* dst = a.out + ((long long)(tok_base + r / a.G) * a.H + (kvh * a.G + r % a.G)) * HD + d;
                    __nv_bfloat162 lo2 = __floats2bfloat162_rn(acc[j].x * inv, acc[j].y * inv), hi2 = __floats2bfloat162_rn(acc[j].z * inv, acc[j].w * inv);
                    uint2 packed;
                    packed.x = *reinterpret_cast<uint32_t*>(&lo2);
                    packed.y = *reinterpret_cast<uint32_t*>(&hi2);
                    *reinterpret_cast<uint2*>(dst) = packed;
                }
            }
        }
        pos += n_here;
        i0 += n_here;
    }
    __syncthreads();
    if (tid == 0 && *gave_up) atomicExch(a.status, 2);
}

// Combine the spans of one (request, kv head) and write the output rows.  grid (K, segments), MERGE_THREADS
// threads.  Each row's span weights exp(m_s - M) go to shared memory first.  A thread then owns four
// neighbouring output elements and every `groups`-th span (groups = threads / owned quadruples, so that all
// threads have work when there are few rows), with its loads independent of one another; the groups' sums
// meet in shared memory and are added in ascending group order, so the result is a fixed function of the
// partials.
#define MERGE_SPANS 64          // spans whose weights fit shared memory at once (longer requests go round again)
#define MERGE_THREADS 512
template <int HD>
__global__ void __launch_bounds__(MERGE_THREADS)
k_attention_merge(AttnMmaArgs a) {
    xr_pdl_launch();
    xr_pdl_wait();
    __shared__ float wgt[16][MERGE_SPANS + 1];
    __shared__ float row_max[16], row_inv[16];
    __shared__ float4 group_sum[MERGE_THREADS];
    const int seg = blockIdx.y, kvh = blockIdx.x;
    const int L = a.seg_len[seg], rows_total = L * a.G;
    if (rows_total > 16) return;
    const int pos0 = a.seg_pos0[seg], tok_base = a.seg_start[seg];
    const int hi_all = pos0 + L - 1;
    const int lo_all = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
    const int SPAN = a.span;
    const int n_spans = hi_all / SPAN - lo_all / SPAN + 1;
    const size_t item0 = ((size_t)seg * a.K + kvh) * a.max_splits;
    const float* ml = a.part_ml + item0 * 32;
    const float* pa = a.part_acc + item0 * 16 * HD;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // one warp per row: maximum and denominator over the spans
    for (int r = warp; r < rows_total; r += MERGE_THREADS / 32) {
        float mm = -INFINITY;
        for (int s = lane; s < n_spans; s += 32) mm = fmaxf(mm, __ldcg(ml + (s * 16 + r) * 2));
        mm = xr_warp_max(mm);
        float off = mm == -INFINITY ? 0.f : mm;
        float ll = 0.f;                      // summed in a fixed order: lane-strided, then the warp tree
        for (int s = lane; s < n_spans; s += 32) ll += __ldcg(ml + (s * 16 + r) * 2 + 1) * expf(__ldcg(ml + (s * 16 + r) * 2) - off);
        ll = xr_warp_sum(ll);
        if (lane == 0) { row_max[r] = off; row_inv[r] = 1.0f / ll; }
    }
    __syncthreads();
    constexpr int QUADS = HD / 4;                       // float4 per row
    const int owned = rows_total * QUADS;               // <= 16 * 32 = MERGE_THREADS
    const int groups = MERGE_THREADS / owned;
    const int g = threadIdx.x / owned, e = threadIdx.x % owned;
    const bool active = g < groups;
    const int r = e / QUADS;
    const float4* src = reinterpret_cast<const float4*>(pa) + e;          // span s: + s * 16 * QUADS
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < n_spans; s0 += MERGE_SPANS) {
        int ns = min(MERGE_SPANS, n_spans - s0);
        for (int i = threadIdx.x; i < rows_total * ns; i += MERGE_THREADS) {
            int rr = i / ns, s = i % ns;
            wgt[rr][s] = expf(__ldcg(ml + ((s0 + s) * 16 + rr) * 2) - row_max[rr]);
        }
        __syncthreads();
        if (active) {
            int s = g;
            for (; s + 3 * groups < ns; s += 4 * groups) {
                float4 v0 = __ldcg(src + (size_t)(s0 + s) * 16 * QUADS);
                float4 v1 = __ldcg(src + (size_t)(s0 + s + groups) * 16 * QUADS);
                float4 v2 = __ldcg(src + (size_t)(s0 + s + 2 * groups) * 16 * QUADS);
                float4 v3 = __ldcg(src + (size_t)(s0 + s + 3 * groups) * 16 * QUADS);
                float w0 = wgt[r][s], w1 = wgt[r][s + groups], w2 = wgt[r][s + 2 * groups], w3 = wgt[r][s + 3 * groups];
                acc.x += v0.x * w0; acc.y += v0.y * w0; acc.z += v0.z * w0; acc.w += v0.w * w0;
                acc.x += v1.x * w1; acc.y += v1.y * w1; acc.z += v1.z * w1; acc.w += v1.w * w1;
                acc.x += v2.x * w2; acc.y += v2.y * w2; acc.z += v2.z * w2; acc.w += v2.w * w2;
                acc.x += v3.x * w3; acc.y += v3.y * w3; acc.z += v3.z * w3; acc.w += v3.w * w3;
            }
            for (; s < ns; s += groups) {
                float4 v = __ldcg(src + (size_t)(s0 + s) * 16 * QUADS);
                float w = wgt[r][s];
                acc.x += v.x * w; acc.y += v.y * w; acc.z += v.z * w; acc.w += v.w * w;
            }
        }
        __syncthreads();
    }
    group_sum[threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.x < owned) {
        float4 t = group_sum[threadIdx.x];
        for (int k = 1; k < groups; k++) {
            float4 u = group_sum[k * owned + threadIdx.x];
            t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
        }
        const float inv = row_inv[r];
        const int d = (e % QUADS) * 4;
        __nv_bfloat16* dst = a.out + ((long long)(tok_base + r / a.G) * a.H + (kvh * a.G + r % a.G)) * HD + d;
        __nv_bfloat162 lo2 = __floats2bfloat162_rn(t.x * inv, t.y * inv), hi2 = __floats2bfloat162_rn(t.z * inv, t.w * inv);
        uint2 packed;
        packed.x = *reinterpret_cast<uint32_t*>(&lo2);
        packed.y = *reinterpret_cast<uint32_t*>(&hi2);
        *reinterpret_cast<uint2*>(dst) = packed;
    }
}

// The same for at most MERGE_SPANS spans per request (what the launcher's span choice gives unless a context is very
// long and alone), in one round of global loads and little code: a kernel this short spends as long fetching its
// instructions as running them, so the rare general case lives in a kernel of its own (k_attention_merge).
template <int HD>
__global__ void __launch_bounds__(MERGE_THREADS)
k_attention_merge_small(AttnMmaArgs a) {
    xr_pdl_launch();
    __shared__ float4 group_sum[MERGE_THREADS];
    // (the step's description does not change while the step runs: it is read before the kernel ahead is complete)
    const int seg = blockIdx.y, kvh = blockIdx.x;
    const int L = a.seg_len[seg], rows_total = L * a.G;
    if (rows_total > 16) return;
    const int pos0 = a.seg_pos0[seg], tok_base = a.seg_start[seg];
    xr_pdl_wait();
    const int hi_all = pos0 + L - 1;
    const int lo_all = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
    const int n_spans = hi_all / a.span - lo_all / a.span + 1;
    const size_t item0 = ((size_t)seg * a.K + kvh) * a.max_splits;
    const float* ml = a.part_ml + item0 * 32;
    const float* pa = a.part_acc + item0 * 16 * HD;
    // The usual case, in one round of global loads: every thread fetches the (maximum, sum) pairs it is to put into
    // shared memory AND the first accumulator quadruples it will weigh, before anything is computed; the rows'
    // maxima and denominators, and then the weights, come from shared memory.
    __shared__ float2 mls[16][MERGE_SPANS];
    constexpr int QUADS = HD / 4;
    const int owned = rows_total * QUADS, groups = MERGE_THREADS / owned;
    const int g = threadIdx.x / owned, e = threadIdx.x % owned, r = e / QUADS;
    const bool active = g < groups;
    const float4* src = reinterpret_cast<const float4*>(pa) + e;
    float2 mine[2];
    const int i0 = threadIdx.x, i1 = threadIdx.x + MERGE_THREADS, n_ml = rows_total * n_spans;      // <= 16 * 64 = 2 * 512
    // (indices clamped so that no load is conditional; xr_ld_now / xr_ld_fence keep them together)
    const int c0 = i0 < n_ml ? i0 : 0, c1 = i1 < n_ml ? i1 : 0;
    mine[0].x = xr_ld_now(ml + ((c0 % n_spans) * 16 + c0 / n_spans) * 2);
    mine[0].y = xr_ld_now(ml + ((c0 % n_spans) * 16 + c0 / n_spans) * 2 + 1);
    mine[1].x = xr_ld_now(ml + ((c1 % n_spans) * 16 + c1 / n_spans) * 2);
    mine[1].y = xr_ld_now(ml + ((c1 % n_spans) * 16 + c1 / n_spans) * 2 + 1);
    float4 v[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
        int sp = g + k * groups;
        v[k] = xr_ld_now4(src + (size_t)(active && sp < n_spans ? sp : 0) * 16 * QUADS);
    }
    xr_ld_fence(mine[0].x); xr_ld_fence(mine[0].y); xr_ld_fence(mine[1].x); xr_ld_fence(mine[1].y);
#pragma unroll
    for (int k = 0; k < 4; k++) xr_ld_fence(v[k]);
    if (i0 < n_ml) mls[i0 / n_spans][i0 % n_spans] = mine[0];
    if (i1 < n_ml) mls[i1 / n_spans][i1 % n_spans] = mine[1];
    __syncthreads();
    // every thread works out its own row's maximum and denominator from shared memory, walking the spans in order
    // (a few dozen at most): cheaper than a phase of its own with a barrier after it, and the same sum in every thread
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float inv = 0.f;
    if (active) {
        float mm = -INFINITY;
        for (int sp = 0; sp < n_spans; sp++) mm = fmaxf(mm, mls[r][sp].x);
        const float off = mm == -INFINITY ? 0.f : mm;
        float ll = 0.f;
        for (int sp = 0; sp < n_spans; sp++) ll += mls[r][sp].y * __expf(mls[r][sp].x - off);
        inv = 1.0f / ll;
#pragma unroll
        for (int k = 0; k < 4; k++) {
            int sp = g + k * groups;
            if (sp < n_spans) {
                float wk = __expf(mls[r][sp].x - off);
                acc.x += v[k].x * wk; acc.y += v[k].y * wk; acc.z += v[k].z * wk; acc.w += v[k].w * wk;
            }
        }
        for (int sp = g + 4 * groups; sp < n_spans; sp += groups) {
            float4 u = __ldcg(src + (size_t)sp * 16 * QUADS);
            float wk = __expf(mls[r][sp].x - off);
            acc.x += u.x * wk; acc.y += u.y * wk; acc.z += u.z * wk; acc.w += u.w * wk;
        }
    }
    group_sum[threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.x < owned) {
        float4 t = group_sum[threadIdx.x];
        for (int k = 1; k < groups; k++) {
            float4 u = group_sum[k * owned + threadIdx.x];
            t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
        }
        const int d = (e % QUADS) * 4;
        __nv_bfloat16* dst = a.out + ((long long)(tok_base + r / a.G) * a.H + (kvh * a.G + r % a.G)) * HD + d;
        __nv_bfloat162 lo2 = __floats2bfloat162_rn(t.x * inv, t.y * inv), hi2 = __floats2bfloat162_rn(t.z * inv, t.w * inv);
        uint2 packed;
        packed.x = *reinterpret_cast<uint32_t*>(&lo2);
        packed.y = *reinterpret_cast<uint32_t*>(&hi2);
        *reinterpret_cast<uint2*>(dst) = packed;
    }
    return;
}

// ---------------------------------------------------------------------------------------------
typedef CUresult (*AttEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static AttEncodeFn att_encode() {
    static AttEncodeFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (AttEncodeFn)ptr;
    }
    return fn;
}

// Even shares are taken when there are more (request, kv head) pairs than CTAs with deep rings fit on the machine.
// Requests of much the same length are better served by spans while one CTA per span is resident at once, three to an
// SM (measured up to 52 requests of 8 kv heads and 8 of 40: 1 to 5 us less than even shares, whose pieces meet through
// global memory); requests of unequal length leave most spans short, and even shares win from about two pairs per
// three SMs on (32 requests of 512 to 4,096 keys: 52.8 against 63.4 us; 12 of 1,024 to 8,192: 46.8 against 59.5 us;
// with 8 such requests a long one is cut into so many pieces that gathering them costs more than the balance gains,
// 38.5 against 33.1 us).
static bool att_even_wanted(long long items, bool uneven) {
    return items > 3LL * xr_sm_count() || (uneven && 8 * items >= 5LL * xr_sm_count());
}
static long long g_even_launches = 0;
// Launches of the even-shares kernel so far (captures count once): lets a test see which kernel a step took.
XR_EXPORT int xr_attention_even_launches() { return (int)(g_even_launches & 0x7fffffff); }
// XRB200_NO_CLUSTER_MERGE=1: spans and the merge kernel only (no exchange inside clusters, no even shares), so that a
// test can compare the bulk-copy kernel with the per-thread copies where both add in the same order.
static bool att_cluster_merge_enabled() {
    static int on = -1;
    if (on < 0) { const char* e = getenv("XRB200_NO_CLUSTER_MERGE"); on = (e && e[0] == '1') ? 0 : 1; }
    return on == 1;
}

// The bulk-copy keys kernel, when the shapes allow it.  Returns 1 if launched (2: and the spans are combined
// already), 0 if not applicable, < 0 on error.
template <int HD>
static int launch_keys_tma(const AttnMmaArgs& a, const void* cache_base, long long n_pages, int n_seg, cudaStream_t stream,
                           int* flags, int n_flags, long long room, bool uneven) {
  if constexpr (HD != 64 && HD != 128) {
    return 0;
  } else {
    if (a.page_shift < 3 || cache_base == nullptr || a.status == nullptr) return 0;
    long long total_rows = n_pages * a.n_layers * 2 * a.K * a.page_size;
    if (total_rows >= (1LL << 31) || ((uintptr_t)cache_base & 15)) return 0;
    AttEncodeFn enc = att_encode();
    if (!enc) return 0;
    CUtensorMap map;
    const unsigned box_rows = (unsigned)(a.page_size < ATT_TILE ? a.page_size : ATT_TILE);
    const XrMapKey key{cache_base, {(unsigned long long)HD, (unsigned long long)total_rows, 0}, {(unsigned long long)HD * 2, 0}, {64, box_rows, 0}, 2, 0};
    if (!xr_cached_map(&map, key, [&](CUtensorMap* out) {
            cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)total_rows};
            cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
            cuuint32_t box[2] = {64, box_rows};
            cuuint32_t estr[2] = {1, 1};
            return enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(cache_base), dims, strides, box, estr,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
        }))
        return -3;
    constexpr int LD = HD + 8;
    constexpr int STAGE = 2 * ATT_TILE * HD * 2, REST = 16 * LD * 2 + 64 + 1024;
    constexpr int RECV = (16 * (HD / 4) + ATT_CLUSTER_MAX) * 16 + ATT_CLUSTER_MAX * 16 * 8 + 16;
    constexpr int S2 = 2 * STAGE + REST, S3 = 3 * STAGE + REST, S4 = 4 * STAGE + REST;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(k_attention_keys_tma<HD, 2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, S2) != cudaSuccess ||
            cudaFuncSetAttribute(k_attention_keys_tma<HD, 3, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, S3) != cudaSuccess ||
            cudaFuncSetAttribute(k_attention_keys_tma<HD, 4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, S4) != cudaSuccess ||
            cudaFuncSetAttribute(k_attention_keys_tma<HD, 2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, S2 + RECV) != cudaSuccess ||
            cudaFuncSetAttribute(k_attention_keys_tma<HD, 3, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, S3 + RECV) != cudaSuccess ||
            cudaFuncSetAttribute(k_attention_keys_tma<HD, 4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, S4 + RECV) != cudaSuccess)
            return XR_ERR_LAUNCH;
        configured = true;
    }
    if (att_even_wanted((long long)n_seg * a.K, uneven) && flags != nullptr && n_seg <= ATT_EVEN_MAX_SEGS && att_cluster_merge_enabled()) {
        // even shares: as many CTAs as are resident at once
        static bool even_configured = false;
        constexpr int EVEN_MAX = 2 * 4 * ATT_TILE * HD * 2 + 16 * LD * 2 + 4 * 16 * HD * 4 + 512 + 64 + 4 * (ATT_EVEN_MAX_SEGS + 4);
        if (!even_configured) {
            if (cudaFuncSetAttribute(k_attention_keys_even<HD, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, EVEN_MAX) != cudaSuccess ||
                cudaFuncSetAttribute(k_attention_keys_even<HD, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, EVEN_MAX) != cudaSuccess ||
                cudaFuncSetAttribute(k_attention_keys_even<HD, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, EVEN_MAX) != cudaSuccess)
                return XR_ERR_LAUNCH;
            even_configured = true;
        }
        const int region = 16 * LD * 2 > 4 * a.recv_rows * HD * 4 ? 16 * LD * 2 : 4 * a.recv_rows * HD * 4;
        const int tail = (region + 512 + 8 * 4 + 4 * (n_seg + 2) + 15) & ~15;
        // the deepest ring with which three CTAs share an SM (measured: three with two stages stream faster than two with
        // three: 128 requests at 704 keys 62.5 against 66.6 us, 48 at 1,500 keys 50.3 against 53.9 us), else two, else one
        auto resident_with = [&](int depth, int bytes) {
            static int known_key[32], known_val[32], known_n = 0;  // asked once per (ring depth, shared memory): the answer does not change
            const int key = bytes * 8 + depth;
            for (int i = 0; i < known_n; i++)
                if (known_key[i] == key) return known_val[i];
            int r = 0;
            cudaError_t e = depth == 4 ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&r, k_attention_keys_even<HD, 4>, ATT_THREADS, bytes)
                          : depth == 3 ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&r, k_attention_keys_even<HD, 3>, ATT_THREADS, bytes)
                                       : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&r, k_attention_keys_even<HD, 2>, ATT_THREADS, bytes);
            if (e != cudaSuccess) { cudaGetLastError(); return 0; }
            if (known_n < 32) { known_key[known_n] = key; known_val[known_n] = r; known_n++; }
            return r;
        };
        int depth = 2, bytes = 2 * STAGE + tail, resident = 0;
        for (int want = 3; want >= 1 && resident == 0; want--)
            for (int d = 4; d >= 2; d--) {
                const int r = resident_with(d, d * STAGE + tail);
                if (r >= want) { depth = d; bytes = d * STAGE + tail; resident = want; break; }
            }
        const long long ctas = (long long)resident * xr_sm_count();
        if (resident >= 1 && ctas <= n_flags && ctas <= room) {
            if (depth == 4) xr_launch((k_attention_keys_even<HD, 4>), dim3((unsigned)ctas), dim3(ATT_THREADS), bytes, stream, map, a, n_seg, flags);
            else if (depth == 3) xr_launch((k_attention_keys_even<HD, 3>), dim3((unsigned)ctas), dim3(ATT_THREADS), bytes, stream, map, a, n_seg, flags);
            else xr_launch((k_attention_keys_even<HD, 2>), dim3((unsigned)ctas), dim3(ATT_THREADS), bytes, stream, map, a, n_seg, flags);
            g_even_launches++;
            return xr_launch_status() == XR_OK ? 2 : XR_ERR_LAUNCH;
        }
    }
    // the fewer CTAs there are, the deeper each one's ring of tiles, so that as many bytes stay in flight per SM
    dim3 grid(a.max_splits, a.K, n_seg);
    long long ctas = (long long)a.max_splits * a.K * n_seg;
    const int depth = ctas <= xr_sm_count() ? 4 : (ctas <= 2 * xr_sm_count() ? 3 : 2);
    // (a single span sends nothing and needs no room to receive; otherwise the room must not cost a resident CTA)
    // what a block receives from the other spans is sized by the step's largest number of packed rows (a decode step:
    // the heads of one group), so that the room seldom costs a resident CTA
    const int recv_sized = (a.recv_rows * (HD / 4) + ATT_CLUSTER_MAX) * 16 + ATT_CLUSTER_MAX * 16 * 8 + 16;
    const int ring = depth == 4 ? S4 : (depth == 3 ? S3 : S2), recv = a.max_splits == 1 ? 0 : (recv_sized < RECV ? recv_sized : RECV);
    const int fit = (227 * 1024) / (ring + 1024), fit_recv = (227 * 1024) / (ring + recv + 1024);
    // (clusters of spans are worth it while all of them are resident at once: with several waves of CTAs the
    // co-scheduling of a cluster's blocks costs more than the merge kernel it saves -- batch 64 at a context of 704:
    // 53 us as clusters of four against 37 + 8 us with the merge kernel)
    (void)fit;
    // (a cluster's blocks lie in one of the machine's eight or so groups of SMs, so each group may leave up to a
    // cluster less one of its slots unused: 8 spans for each of 32 (request, kv head) pairs are 256 blocks for 296
    // slots, and inside a step, where a few slots are still held by the kernels around it, some clusters waited for
    // others to end -- 131,072 keys, 4 requests: 16.8 ms a step against 14.7 with 5 spans each)
    const long long packing = 8LL * (a.max_splits - 1);
    if (a.max_splits <= ATT_CLUSTER_MAX && att_cluster_merge_enabled() && (a.max_splits == 1 || ctas + packing <= (long long)fit_recv * xr_sm_count())) {
        // the spans of a request as one cluster, which also combines them (returns 2: no merge kernel is to follow)
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid; cfg.blockDim = dim3(ATT_THREADS); cfg.stream = stream;
        cfg.dynamicSmemBytes = ring + recv;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = a.max_splits; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = xr_pdl_enabled() ? 2 : 1;
        if (depth == 4) cudaLaunchKernelEx(&cfg, k_attention_keys_tma<HD, 4, true>, map, a);
        else if (depth == 3) cudaLaunchKernelEx(&cfg, k_attention_keys_tma<HD, 3, true>, map, a);
        else cudaLaunchKernelEx(&cfg, k_attention_keys_tma<HD, 2, true>, map, a);
        return xr_launch_status() == XR_OK ? 2 : XR_ERR_LAUNCH;
    }
    if (depth == 4)
        xr_launch((k_attention_keys_tma<HD, 4, false>), dim3(grid), dim3(ATT_THREADS), S4, stream, map, a);
    else if (depth == 3)
        xr_launch((k_attention_keys_tma<HD, 3, false>), dim3(grid), dim3(ATT_THREADS), S3, stream, map, a);
    else
        xr_launch((k_attention_keys_tma<HD, 2, false>), dim3(grid), dim3(ATT_THREADS), S2, stream, map, a);
    return xr_launch_status() == XR_OK ? 1 : XR_ERR_LAUNCH;
  }
}

template <int HD>
static int launch_attention(const AttnMmaArgs& a, int n_seg, int max_seg_len, int max_kv_len, int any_short, int any_long,
                            const void* cache_base, long long n_pages, cudaStream_t stream, int* flags, int n_flags, long long room, bool uneven,
                            long long row_tiles) {
    constexpr int LD = HD + 8;
    constexpr int SMEM_ROWS = (ATT_ROWS + 4 * ATT_TILE) * LD * 2;
    constexpr int KEYS_MERGE = 16 * LD * 2 + (4 * 16 * HD + 4 * 16 * 2) * 4;
    constexpr int KEYS_TILES2 = (16 + 2 * 2 * ATT_TILE) * LD * 2, KEYS_TILES4 = (16 + 2 * 4 * ATT_TILE) * LD * 2;
    constexpr int SMEM_KEYS2 = KEYS_TILES2 > KEYS_MERGE ? KEYS_TILES2 : KEYS_MERGE;
    constexpr int SMEM_KEYS4 = KEYS_TILES4 > KEYS_MERGE ? KEYS_TILES4 : KEYS_MERGE;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(k_attention_rows<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_ROWS) != cudaSuccess ||
            cudaFuncSetAttribute(k_attention_keys<HD, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_KEYS2) != cudaSuccess ||
            cudaFuncSetAttribute(k_attention_keys<HD, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_KEYS4) != cudaSuccess)
            return XR_ERR_LAUNCH;
        configured = true;
    }
    if (any_long) {
        // row_tiles: the 64-row tiles of the portions with more than 16 packed rows, summed; 0: not known, and an upper
        // bound is taken (blocks beyond the true number return at once)
        long long tiles = row_tiles > 0 ? row_tiles : (((long long)max_seg_len * a.G + ATT_ROWS - 1) / ATT_ROWS) * n_seg;
        if (tiles > 0x7fffffffLL || n_seg > 65535 || a.K > 65535) return XR_ERR_ARG;
        xr_launch((k_attention_rows<HD>), dim3((unsigned)tiles, a.K, 1), dim3(ATT_THREADS), SMEM_ROWS, stream, a, n_seg);
        int rc = xr_launch_status();
        if (rc != XR_OK) return rc;
    }
    if (any_short) {
        if (n_seg > 65535 || a.K > 65535) return XR_ERR_ARG;
        int tma = launch_keys_tma<HD>(a, cache_base, n_pages, n_seg, stream, flags, n_flags, room, uneven);
        if (tma < 0) return tma;
        // few CTAs (small batch): deeper stages; many: more CTAs per SM.  The arithmetic is the same.
        if (tma == 2) return XR_OK;                    // the spans were combined inside the clusters
        if (tma == 1) {
        } else if ((long long)a.max_splits * a.K * n_seg <= 2 * xr_sm_count())
            xr_launch((k_attention_keys<HD, 4>), dim3(a.max_splits, a.K, n_seg), dim3(ATT_THREADS), SMEM_KEYS4, stream, a);
        else
            xr_launch((k_attention_keys<HD, 2>), dim3(a.max_splits, a.K, n_seg), dim3(ATT_THREADS), SMEM_KEYS2, stream, a);
        int rc = xr_launch_status();
        if (rc != XR_OK) return rc;
        if (a.max_splits <= MERGE_SPANS) xr_launch((k_attention_merge_small<HD>), dim3(a.K, n_seg), dim3(MERGE_THREADS), 0, stream, a);
        else xr_launch((k_attention_merge<HD>), dim3(a.K, n_seg), dim3(MERGE_THREADS), 0, stream, a);
        return xr_launch_status();
    }
    return XR_OK;
}

// Slots of scratch per (request, kv head) pair that a step needs: the spans the keys kernel cuts a longest key range of
// `max_kv_len` into (window > 0: at most that many keys), or, where even shares are taken, one slot per CTA.
// `items`: (request, kv head) pairs of the step, n_seg * K.
static int att_spans(int max_kv_len, int window, long long items) {
    int range = att_range(max_kv_len, window);
    int span = att_choose_span(range, items);
    return (range + span - 1) / span + (window > 0 ? 1 : 0);
}
XR_EXPORT int xr_attention_mma_splits(int max_kv_len, int window, long long items) {
    int need = att_spans(max_kv_len, window, items);
    if (items >= 1 && att_even_wanted(items, true)) {
        long long per = (3LL * xr_sm_count() + items - 1) / items;
        if (per > need) need = (int)per;
    }
    return need;
}

// part_acc: float32 [n_seg * K * splits * 16 * hd], part_ml: float32 [n_seg * K * splits * 32]
// (only read and written when any_short).  splits: at least xr_attention_mma_splits(max_kv_len, window, n_seg * K).
// flags: n_flags zeroed words that only this kernel touches (it leaves them zero), or null.
// uneven: the requests' key ranges differ much in length (a hint for the choice between spans and even shares).
// row_tiles: the 64-row tiles of the portions with more than 16 packed rows, summed, or 0 if the caller does not know.
XR_EXPORT int xr_attention_mma(const void* q, void* out, const void* cache_k, const int* seg_start, const int* seg_len,
                               const int* seg_pos0, const int* block_tables, float* part_acc, float* part_ml,
                               long long q_stride, long long page_stride, long long v_offset, int n_seg, int H, int K,
                               int hd, int max_pages, int page_size, int window, float scale, int max_seg_len,
                               int max_kv_len, int splits, int any_short, int any_long, const void* cache_base,
                               long long n_pages, int n_layers, int layer, int* status, int* flags, int n_flags,
                               int uneven, long long row_tiles, cudaStream_t stream) {
    if (n_seg < 1 || H < 1 || K < 1 || H % K != 0 || hd < 16 || hd > 128 || hd % 16 != 0 || page_size < 1 || window < 0 ||
        (q_stride % 8) != 0 || ((uintptr_t)q & 15) || ((uintptr_t)cache_k & 15) || (page_stride % 8) != 0 || (v_offset % 8) != 0)
        return XR_ERR_ARG;
    if (H / K > 16 && any_short) return XR_ERR_ARG;     // more heads per group than one instruction tile holds
    const int spans = att_spans(max_kv_len, window, (long long)n_seg * K);
    if (any_short && splits < spans) return XR_ERR_ARG;
    AttnMmaArgs a{(const __nv_bfloat16*)q, (__nv_bfloat16*)out, (const __nv_bfloat16*)cache_k, seg_start, seg_len, seg_pos0,
                  block_tables, part_acc, part_ml, q_stride, page_stride, v_offset, H, K, H / K, max_pages, page_size, window,
                  spans, 0, scale, -1, n_layers, layer, status, 16};
    { long long rows = (long long)(max_seg_len < 1 ? 1 : max_seg_len) * a.G; a.recv_rows = rows < 16 ? (int)rows : 16; }
    a.span = att_choose_span(att_range(max_kv_len, window), (long long)n_seg * K);
    const long long room = (long long)splits * n_seg * K;
    if ((page_size & (page_size - 1)) == 0) { int sh = 0; while ((1 << sh) < page_size) sh++; a.page_shift = sh; }
    switch (hd) {
        case 16: return launch_attention<16>(a, n_seg, max_seg_len, max_kv_len, any_short, any_long, cache_base, n_pages, stream, flags, n_flags, room, uneven != 0, row_tiles);
        case 32: return launch_attention<32>(a, n_seg, max_seg_len, max_kv_len, any_short, any_long, cache_base, n_pages, stream, flags, n_flags, room, uneven != 0, row_tiles);
        case 48: return launch_attention<48>(a, n_seg, max_seg_len, max_kv_len, any_short, any_long, cache_base, n_pages, stream, flags, n_flags, room, uneven != 0, row_tiles);
        case 64: return launch_attention<64>(a, n_seg, max_seg_len, max_kv_len, any_short, any_long, cache_base, n_pages, stream, flags, n_flags, room, uneven != 0, row_tiles);
        case 80: return launch_attention<80>(a, n_seg, max_seg_len, max_kv_len, any_short, any_long, cache_base, n_pages, stream, flags, n_flags, room, uneven != 0, row_tiles);
        case 96: return launch_attention<96>(a, n_seg, max_seg_len, max_kv_len, any_short, any_long, cache_base, n_pages, stream, flags, n_flags, room, uneven != 0, row_tiles);
        case 112: return launch_attention<112>(a, n_seg, max_seg_len, max_kv_len, any_short, any_long, cache_base, n_pages, stream, flags, n_flags, room, uneven != 0, row_tiles);
        case 128: return launch_attention<128>(a, n_seg, max_seg_len, max_kv_len, any_short, any_long, cache_base, n_pages, stream, flags, n_flags, room, uneven != 0, row_tiles);
    }
    return XR_ERR_ARG;
}
