// Picking the next token from float32 logits on the device, in two launches: the reference's short cuts, one block per
// row (k_sample with shortcuts: top-k by selection, else the head of the distribution), then, for the rows they left
// open (usually none: the launch then reads a word a row and ends), the long way by threshold descents -- spread over a
// cluster of eight blocks per row that keeps the row in registers when the rows are few and have more than 1,024
// values (k_sample_cluster, further down), else one block per row.  And the log-probability of a given token per row
// (k_logprob, at the end).
//
// The chain is the reference's `sample_pick` (src/sample.c:141-329) with
// `pick_scaled` (src/sample.c:86-127):
//   1. temp > 0 and repeat_penalty != 1: for each recent token, logit > 0 ? logit / pen : logit * pen;
//   2. temp <= 0: the argmax, first index on ties, no penalty;
//   3. v = logit / temp; candidates ordered by (v descending, id ascending);
//   4. top-k keeps the first k; softmax over the survivors;
//   5. top-p keeps the shortest prefix whose probability reaches top_p; renormalise;
//   6. min-p drops candidates below min_p * p_max; renormalise;
//   7. the pick is the first candidate whose cumulative probability exceeds r (a uniform draw
//      in [0, 1) that the host makes from the request's own xorshift64 state, src/sample.c:13-20).
// The long way never sorts.  Every cut above is a prefix of the same order, so it
// is described by a threshold in an order-preserving integer image of v (plus, among exact ties, a
// count of ids).  Thresholds are found by descending over the 32 key bits, two bits a pass (three
// candidate thresholds, each with its own block-wide sum in a fixed order, which makes the result
// deterministic); a pass reads the row in runs of eight 16-byte loads per thread.
#include "common.cuh"
#include <math.h>

#define SMP_THREADS 1024
#define SMP_RECENT 256
#define SMP_EXEMPT 8          // ids per row that the window never holds

struct SampleArgs {
    const float* logits;      // [rows, ld]
    long long ld;
    int V;
    const float* temp;        // per row
    const int* top_k;
    const float* top_p;
    const float* min_p;
    const float* penalty;
    const float* draw;        // r per row
    const int* recent;        // [rows, SMP_RECENT], entries < 0 are empty
    int* out;                 // [rows]
    // A step may be queued before the host has read the token that the step before it sampled.  That token belongs in
    // the window all the same: pending[3 row] is where it lies in `feed` (or -1: the window is complete),
    // pending[3 row + 1] the window entry it takes, pending[3 row + 2] how many of exempt[SMP_EXEMPT row ..] count:
    // ids that the window never holds (src/sample.c:159-162), which the host cannot strike out of a token it has not seen.
    const int* pending;       // [rows, 3] or null
    const int* feed;
    const int* exempt;        // [rows, SMP_EXEMPT]
    // Rows that the short cuts left open: row r is wanted iff todo[r * todo_stride] != 0 (null: every row).  The kernel of
    // the short cuts writes these words, the kernels of the long way only read them.
    const int* todo;
    long long todo_stride;
};

// Entry j of a row's window of recent tokens.
__device__ __forceinline__ int smp_window_entry(const SampleArgs& a, int row, int j) {
    int tok = a.recent[(size_t)row * SMP_RECENT + j];
    if (a.pending != nullptr && a.pending[3 * row] >= 0 && a.pending[3 * row + 1] == j) {
        tok = a.feed[a.pending[3 * row]];
        for (int e = 0; e < a.pending[3 * row + 2] && e < SMP_EXEMPT; e++)
            if (a.exempt[row * SMP_EXEMPT + e] == tok) tok = -1;
    }
    return tok;
}

__device__ __forceinline__ unsigned xr_key(float v) {
    unsigned u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);      // larger float <=> larger key
}

// block-wide sums in a fixed order (threads -> warps -> warp 0)
__device__ __forceinline__ double blk_sum_d(double v, double* sh) {
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    if (warp == 0) {
        double t = lane < (SMP_THREADS / 32) ? sh[lane] : 0.0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) sh[32] = t;
    }
    __syncthreads();
    return sh[32];
}
__device__ __forceinline__ long long blk_sum_ll(long long v, double* sh) {
    long long* s = (long long*)sh;
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) s[warp] = v;
    __syncthreads();
    if (warp == 0) {
        long long t = lane < (SMP_THREADS / 32) ? s[lane] : 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) s[32] = t;
    }
    __syncthreads();
    return s[32];
}

// The same sums for three values at once (one pass of a descent weighs three candidate thresholds).
__device__ __forceinline__ void blk_sum3_d(double (&v)[3], double* sh) {
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int j = 0; j < 3; j++)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v[j] += __shfl_xor_sync(0xffffffffu, v[j], o);
    __syncthreads();
    if (lane == 0) { sh[warp * 3] = v[0]; sh[warp * 3 + 1] = v[1]; sh[warp * 3 + 2] = v[2]; }
    __syncthreads();
    if (warp < 3) {
        double t = lane < (SMP_THREADS / 32) ? sh[lane * 3 + warp] : 0.0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) sh[100 + warp] = t;
    }
    __syncthreads();
    v[0] = sh[100]; v[1] = sh[101]; v[2] = sh[102];
}
__device__ __forceinline__ void blk_sum3_ll(long long (&v)[3], double* sh) {
    long long* s = (long long*)sh;
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int j = 0; j < 3; j++)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v[j] += __shfl_xor_sync(0xffffffffu, v[j], o);
    __syncthreads();
    if (lane == 0) { s[warp * 3] = v[0]; s[warp * 3 + 1] = v[1]; s[warp * 3 + 2] = v[2]; }
    __syncthreads();
    if (warp < 3) {
        long long t = lane < (SMP_THREADS / 32) ? s[lane * 3 + warp] : 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) s[100 + warp] = t;
    }
    __syncthreads();
    v[0] = s[100]; v[1] = s[101]; v[2] = s[102];
}

// f(i, vals[i]) for every i of the row.  A row is half a megabyte that one block reads alone, many times: eight
// 16-byte loads a thread are issued as one run, so a pass takes a few trips to L2 instead of dozens.  (A row that
// does not start on a 16-byte boundary -- an odd vocabulary -- is read element by element.)
template <typename F>
__device__ __forceinline__ void smp_for_each(const float* vals, int V, F f) {
    const int tid = threadIdx.x;
    int done = 0;
    if ((((uintptr_t)vals) & 15) == 0) {
        const float4* v4 = reinterpret_cast<const float4*>(vals);
        const int quads = V >> 2;
        for (int q0 = 0; q0 < quads; q0 += 8 * SMP_THREADS) {
            float4 v[8];
#pragma unroll
            for (int k = 0; k < 8; k++) {
                int q = q0 + k * SMP_THREADS + tid;
                v[k] = xr_ld_now4(v4 + (q < quads ? q : quads - 1));
            }
#pragma unroll
            for (int k = 0; k < 8; k++) xr_ld_fence(v[k]);
#pragma unroll
            for (int k = 0; k < 8; k++) {
                int q = q0 + k * SMP_THREADS + tid;
                if (q < quads) { f(4 * q, v[k].x); f(4 * q + 1, v[k].y); f(4 * q + 2, v[k].z); f(4 * q + 3, v[k].w); }
            }
        }
        done = quads << 2;
    }
    for (int i = done + tid; i < V; i += SMP_THREADS) f(i, vals[i]);
}

// The set of surviving candidates: key > thr, or key == thr and fewer than `n_eq` equal keys have
// a smaller id.  n_eq < 0 keeps every equal key.
struct Cut { unsigned thr; long long n_eq; };

// id such that exactly `n` candidates with key == thr have an id below it (ids ascending).
__device__ int nth_equal_id(int V, const float* vals, unsigned thr, long long n, double* sh) {
    // each thread owns a contiguous id range, so a prefix over threads is a prefix over ids
    int per = (V + SMP_THREADS - 1) / SMP_THREADS;
    int lo = threadIdx.x * per, hi = min(V, lo + per);
    long long mine = 0;
    for (int i = lo; i < hi; i++) mine += (xr_key(vals[i]) == thr);
    long long* s = (long long*)sh + 40;
    __syncthreads();
    s[threadIdx.x] = mine;
    __syncthreads();
    __shared__ int found;
    if (threadIdx.x == 0) {
        long long run = 0; int f = V;
        for (int t = 0; t < SMP_THREADS; t++) {
            if (run + s[t] > n) {       // the n-th (0-based) equal lies in thread t's range
                int a = t * per, b = min(V, a + per);
                long long c = run;
                for (int i = a; i < b; i++) if (xr_key(vals[i]) == thr) { if (c == n) { f = i; break; } c++; }
                break;
            }
            run += s[t];
        }
        found = f;
    }
    __syncthreads();
    return found;
}

// argmax of a row, first index on ties (src/sample.c:169-172), by one block.  A row is half a megabyte that the block
// reads alone: eight 16-byte loads a thread are issued as one run, so the row takes a few trips to L2, not dozens.
__device__ __forceinline__ void smp_argmax(const float* lg, int V, int* out, float* sh_f, int* sh_i) {
    const int tid = threadIdx.x;
    float best = -INFINITY; int bi = 0x7fffffff;
    int done = 0;
    if ((((uintptr_t)lg) & 15) == 0) {
        const float4* lg4 = reinterpret_cast<const float4*>(lg);
        const int quads = V >> 2;
        for (int q0 = 0; q0 < quads; q0 += 8 * SMP_THREADS) {
            float4 v[8];
#pragma unroll
            for (int k = 0; k < 8; k++) {
                int q = q0 + k * SMP_THREADS + tid;
                v[k] = xr_ld_now4(lg4 + (q < quads ? q : quads - 1));
            }
#pragma unroll
            for (int k = 0; k < 8; k++) xr_ld_fence(v[k]);
#pragma unroll
            for (int k = 0; k < 8; k++) {
                int q = q0 + k * SMP_THREADS + tid;
                if (q < quads) {
                    // ascending indices within the thread, so `>` alone keeps the first of equal values
                    int i = q << 2;
                    if (v[k].x > best) { best = v[k].x; bi = i; }
                    if (v[k].y > best) { best = v[k].y; bi = i + 1; }
                    if (v[k].z > best) { best = v[k].z; bi = i + 2; }
                    if (v[k].w > best) { best = v[k].w; bi = i + 3; }
                }
            }
        }
        done = quads << 2;
    }
    for (int i = done + tid; i < V; i += SMP_THREADS) {
        float x = lg[i];
        if (x > best || (x == best && i < bi)) { best = x; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ob = __shfl_xor_sync(0xffffffffu, best, o); int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if ((tid & 31) == 0) { sh_f[tid >> 5] = best; sh_i[tid >> 5] = bi; }
    __syncthreads();
    if (tid < 32) {
        best = sh_f[tid]; bi = sh_i[tid];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ob = __shfl_xor_sync(0xffffffffu, best, o); int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        if (tid == 0) *out = bi == 0x7fffffff ? 0 : bi;
    }
}

// The reference does not sort the vocabulary either when it can help it (src/sample.c:177-307): with top-k it selects
// the k largest and sorts those; without, it gathers the head of the distribution (candidates within a factor of 1,024
// of the best, loosened up to five times) and uses it once the head provably holds every survivor: top_p of the whole
// mass, or everything above the min-p floor, or more mass than the draw needs.  The sorted candidates then go through
// `pick_scaled` (src/sample.c:86-127) in float32, one after the other.  The same short cuts here: candidates are
// gathered into shared memory, put in order by counting (key descending, id ascending), and the chain runs on them
// with the reference's own arithmetic.  A row whose head does not fit, or is never enough, or whose walk runs off the
// head's end, is left open for the long way (the threshold descents, launched behind this kernel), which needs no room
// and no sort.
#define SMP_CAP 4096               // candidates that fit (the reference's HEAD_CAP)
#define SMP_DYN_MAX (160 * 1024)   // shared memory the short cuts may ask for: the candidates and one bit per token id
#define SMP_KMAX 1024              // largest top-k selected this way: the k-th largest of the threads' maxima bounds the k-th largest of the row

__device__ __forceinline__ float smp_key_value(unsigned k) { return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k); }

// Put the n gathered (key, id) in order and keep the first `keep`: s_p[rank] = value, s_id[rank] = id.
__device__ __forceinline__ void smp_order(const unsigned* c_key, const int* c_id, int n, int keep, float* s_p, int* s_id) {
    for (int j = threadIdx.x; j < n; j += SMP_THREADS) {
        const unsigned kj = c_key[j];
        const int ij = c_id[j];
        int rank = 0;
        for (int i = 0; i < n; i++) rank += (c_key[i] > kj) || (c_key[i] == kj && c_id[i] < ij);
        if (rank < keep) { s_p[rank] = smp_key_value(kj); s_id[rank] = ij; }
    }
    __syncthreads();
}

// `pick_scaled` on m candidates in order (values in s_p, overwritten by their probabilities).  norm_sum > 0: the
// whole vocabulary's sum of exponentials, which then is the denominator.  Returns the pick, or -1 if the walk ran off
// the end of a head (norm_sum > 0).  Divisions are spread over the threads; every sum runs in one thread, in order.
__device__ int smp_pick_scaled(float* s_p, const int* s_id, int m, float norm_sum, float top_p, float min_p, float r, float* bc_f, int* bc_i) {
    const int tid = threadIdx.x;
    const float top = s_p[0];
    __syncthreads();
    for (int i = tid; i < m; i += SMP_THREADS) s_p[i] = expf(s_p[i] - top);
    __syncthreads();
    if (tid == 0) {
        float sum = 0.f;
        for (int i = 0; i < m; i++) sum += s_p[i];
        *bc_f = norm_sum > 0.f ? norm_sum : sum;
    }
    __syncthreads();
    for (int i = tid; i < m; i += SMP_THREADS) s_p[i] /= *bc_f;
    __syncthreads();
    int k = m;
    if (top_p < 1.0f) {
        if (tid == 0) {
            float cum = 0.f;
            int cut = k;
            for (int i = 0; i < k; i++) { cum += s_p[i]; if (cum >= top_p) { cut = i + 1; break; } }
            cum = 0.f;
            for (int i = 0; i < cut; i++) cum += s_p[i];
            *bc_i = cut; *bc_f = cum;
        }
        __syncthreads();
        k = *bc_i;
        for (int i = tid; i < k; i += SMP_THREADS) s_p[i] /= *bc_f;
        __syncthreads();
    }
    if (min_p > 0.0f) {
        if (tid == 0) {
            const float floor_p = min_p * s_p[0];
            int cut = k;
            for (int i = 1; i < k; i++) if (s_p[i] < floor_p) { cut = i; break; }
            float cum = 0.f;
            for (int i = 0; i < cut; i++) cum += s_p[i];
            *bc_i = cut; *bc_f = cum;
        }
        __syncthreads();
        if (*bc_i < k) {
            k = *bc_i;
            for (int i = tid; i < k; i += SMP_THREADS) s_p[i] /= *bc_f;
        }
        __syncthreads();
    }
    if (tid == 0) {
        float cum = 0.f;
        int pick = s_id[k - 1];
        bool hit = false;
        for (int i = 0; i < k; i++) { cum += s_p[i]; if (r < cum) { pick = s_id[i]; hit = true; break; } }
        *bc_i = (hit || norm_sum <= 0.f) ? pick : -1;
    }
    __syncthreads();
    return *bc_i;
}

__global__ void __launch_bounds__(SMP_THREADS)
k_sample(SampleArgs a, float* scratch /* [rows, V] scaled values, or null when nothing needs them */, int shortcuts /* 1: the short cuts and nothing else */) {
    xr_pdl_launch();
    extern __shared__ __align__(16) uint8_t smp_dyn[];          // short cuts: [SMP_CAP] keys, ids, values in order, ids in order; window bits
    __shared__ double sh[40 + SMP_THREADS];
    __shared__ float sh_f[33];
    __shared__ int sh_i[33];
    int row = blockIdx.x, tid = threadIdx.x;
    const float* lg = a.logits + (size_t)row * a.ld;
    // (the rows' parameters are written before the step's kernels are queued: they may be read before the wait)
    float temp = a.temp[row];
    int V = a.V;
    xr_pdl_wait();
    if (a.todo != nullptr && !shortcuts) {
        // the long way after the short cuts: only for the rows they left open (the word lies where this row is staged
        // below: everyone has read it before anyone writes there)
        const int wanted = a.todo[(size_t)row * a.todo_stride];
        __syncthreads();
        if (!wanted) return;
    }
    int* todo_word = shortcuts ? const_cast<int*>(a.todo) + (size_t)row * a.todo_stride : nullptr;

    if (temp <= 0.f) { smp_argmax(lg, V, a.out + row, sh_f, sh_i); if (todo_word && tid == 0) *todo_word = 0; return; }

    if (shortcuts) {
        // Nothing is staged here: a pass reads the logits and works out each value again, logit -> penalised (once per
        // occurrence in the window) -> / temp, the same operations in the same order as the staging below.
        unsigned* c_key = (unsigned*)smp_dyn;
        int* c_id = (int*)(c_key + SMP_CAP);
        float* s_p = (float*)(c_id + SMP_CAP);
        int* s_id = (int*)(s_p + SMP_CAP);
        unsigned* in_window = (unsigned*)(s_id + SMP_CAP);          // one bit per token id: it is in the window of recent tokens
        __shared__ int rec_s[SMP_RECENT];
        __shared__ int n_cand, bc_i;
        __shared__ unsigned bound;
        __shared__ float bc_f;
        const float pen = a.penalty[row];
        const bool penalised = a.recent != nullptr && pen != 1.0f;
        if (penalised) {
            for (int w = tid; w < (V + 31) / 32; w += SMP_THREADS) in_window[w] = 0u;
            if (tid < SMP_RECENT) rec_s[tid] = smp_window_entry(a, row, tid);
            __syncthreads();
            if (tid < SMP_RECENT) { const int tok = rec_s[tid]; if (tok >= 0 && tok < V) atomicOr(&in_window[tok >> 5], 1u << (tok & 31)); }
            __syncthreads();
        }
        auto value_of = [&](int i, float x) {
            if (penalised && ((in_window[i >> 5] >> (i & 31)) & 1u)) {
                int cnt = 0;
                for (int j = 0; j < SMP_RECENT; j++) cnt += rec_s[j] == i;
                for (int c = 0; c < cnt; c++) x = x > 0.f ? x / pen : x * pen;
            }
            return x / temp;
        };
        // The largest value.  Dividing by a positive temperature keeps the order, so outside the window the largest value
        // is the largest logit's; the window's few tokens are worked out one by one.  A thread asks whether a token is
        // in the window only when it would be the thread's new maximum.
        auto in_win = [&](int i) { return penalised && ((in_window[i >> 5] >> (i & 31)) & 1u) != 0u; };
        float traw = -INFINITY;                                     // this thread's largest logit outside the window
        smp_for_each(lg, V, [&](int i, float x) { if (x > traw && !in_win(i)) traw = x; });
        float wv = -INFINITY;                                       // this thread's window token, if it has one: its value
        int wtok = -1;
        if (penalised && tid < SMP_RECENT) {
            const int tok = rec_s[tid];
            if (tok >= 0 && tok < V) {
                bool first = true;
                for (int j = 0; j < tid; j++) first = first && rec_s[j] != tok;
                if (first) { wtok = tok; wv = value_of(tok, lg[tok]); }
            }
        }
        float mx = xr_warp_max(fmaxf(traw / temp, wv));
        if ((tid & 31) == 0) sh_f[tid >> 5] = mx;
        __syncthreads();
        if (tid < 32) { float t = sh_f[tid]; t = xr_warp_max(t); if (tid == 0) sh_f[32] = t; }
        __syncthreads();
        mx = sh_f[32];
        __syncthreads();
        const int top_k = a.top_k[row];
        const float top_p = a.top_p[row], min_p = a.min_p[row], r = a.draw[row];
        int m = 0;                     // candidates in order, if a short cut applies
        float norm_sum = 0.f;
        if (top_k > 0 && top_k < V && top_k <= SMP_KMAX) {
            // The k largest of the threads' maxima are k tokens outside the window: the k-th largest of them is a lower
            // bound of the row's k-th largest value, and usually few values lie above it.  A logit a shade below the bound
            // may still round to the bound's value when divided, and then its id decides: the comparison that costs
            // nothing lets those through, the one on the values is exact.
            unsigned* tm = (unsigned*)s_id;
            tm[tid] = xr_key(traw);
            if (tid == 0) n_cand = 0;
            __syncthreads();
            // (the maxima of the first 8 k threads will do: their k-th largest is a bound all the same, somewhat lower, and
            // ranking a few hundred keys against each other is quick where ranking all 1,024 costs more than a pass)
            const int ranked = min(SMP_THREADS, max(128, 8 * top_k));
            if (tid < ranked) {
                const unsigned my = tm[tid];
                int rank = 0;
                for (int j = 0; j < ranked; j++) rank += (tm[j] > my) || (tm[j] == my && j < tid);
                if (rank == top_k - 1) bound = my;
            }
            __syncthreads();
            const float bound_x = smp_key_value(bound);
            const float lo = bound_x - fabsf(bound_x) * 1e-6f - 1e-30f;
            const unsigned lowest = xr_key(bound_x / temp);
            smp_for_each(lg, V, [&](int i, float x) {
                if (x >= lo && !in_win(i)) {
                    const unsigned k = xr_key(x / temp);
                    if (k >= lowest) { const int at = atomicAdd(&n_cand, 1); if (at < SMP_CAP) { c_key[at] = k; c_id[at] = i; } }
                }
            });
            if (wtok >= 0 && xr_key(wv) >= lowest) { const int at = atomicAdd(&n_cand, 1); if (at < SMP_CAP) { c_key[at] = xr_key(wv); c_id[at] = wtok; } }
            __syncthreads();
            const int nc = n_cand;
            if (nc >= top_k && nc <= SMP_CAP) { smp_order(c_key, c_id, nc, top_k, s_p, s_id); m = top_k; }
        } else if (!(top_k > 0 && top_k < V) && V >= 4096) {
            // the whole mass and the first head in one pass; a head that is not enough costs a pass per loosening
            float t_log = logf(1.0f / 1024.0f);
            double total = 0.0;
            for (int loosen = 0; loosen < 6; loosen++, t_log *= 4.f) {
                if (tid == 0) n_cand = 0;
                __syncthreads();
                double head = 0.0, all = 0.0;
                smp_for_each(lg, V, [&](int i, float x) {
                    const float v = value_of(i, x);
                    const float e = expf(v - mx);
                    if (loosen == 0) all += (double)e;
                    if (v - mx >= t_log) {
                        const int at = atomicAdd(&n_cand, 1);
                        if (at < SMP_CAP) { c_key[at] = xr_key(v); c_id[at] = i; }
                        head += (double)e;
                    }
                });
                if (loosen == 0) total = blk_sum_d(all, sh);
                head = blk_sum_d(head, sh);
                const int nc = n_cand;
                if (nc > SMP_CAP) break;                           // the head is too broad
                const bool enough = top_p < 1.0f ? head >= (double)top_p * total
                                  : (min_p > 0.0f ? t_log <= logf(min_p) : head > (double)r * total);
                // (a head of hundreds that is not enough belongs to a flat row: four times the distance in the logarithm
                // takes in most of the vocabulary, so the pass that would find that out is spared)
                if (!enough && nc > SMP_CAP / 8) break;
                if (!enough) { __syncthreads(); continue; }
                smp_order(c_key, c_id, nc, nc, s_p, s_id);
                m = nc; norm_sum = (float)total;
                break;
            }
        }
        int pick = -1;
        if (m > 0) pick = smp_pick_scaled(s_p, s_id, m, norm_sum, top_p, min_p, r, &bc_f, &bc_i);
        if (tid == 0) {
            if (pick >= 0) a.out[row] = pick;
            *todo_word = pick >= 0 ? 0 : 1;          // open: the kernel of the long way, queued behind this one, takes the row
        }
        return;
    }

    // Stage the row: copy, penalise the recent tokens (once per occurrence in the window, as the
    // reference's loop does, src/sample.c:148-166), then scale by 1/temp.  Later passes read the
    // staged values back, so every pass sees the same numbers.
    float* vals = scratch + (size_t)row * V;
    smp_for_each(lg, V, [&](int i, float v) { vals[i] = v; });
    __syncthreads();
    float pen = a.penalty[row];
    if (a.recent != nullptr && pen != 1.0f) {
        __shared__ int rec[SMP_RECENT];
        if (tid < SMP_RECENT) rec[tid] = smp_window_entry(a, row, tid);
        __syncthreads();
        if (tid < SMP_RECENT) {
            int tok = rec[tid];
            if (tok >= 0 && tok < V) {
                bool first = true; int cnt = 0;
                for (int j = 0; j < SMP_RECENT; j++) { if (rec[j] == tok) { cnt++; if (j < tid) first = false; } }
                if (first) {
                    float x = vals[tok];
                    for (int c = 0; c < cnt; c++) x = x > 0.f ? x / pen : x * pen;
                    vals[tok] = x;
                }
            }
        }
    }
    __syncthreads();
    float mx = -INFINITY;
    smp_for_each(vals, V, [&](int i, float x) {
        float v = x / temp;
        vals[i] = v;
        mx = fmaxf(mx, v);
    });
    mx = xr_warp_max(mx);
    if ((tid & 31) == 0) sh_f[tid >> 5] = mx;
    __syncthreads();
    if (tid < 32) { float t = sh_f[tid]; t = xr_warp_max(t); if (tid == 0) sh_f[32] = t; }
    __syncthreads();
    mx = sh_f[32];
    __syncthreads();

    int top_k = a.top_k[row];
    Cut cut{0u, -1};               // everything survives
    // ---- top-k: the k-th largest key by descending over the key bits with counts ----
    if (top_k > 0 && top_k < V) {
        unsigned thr = 0;
        for (int shift = 30; shift >= 0; shift -= 2) {
            const unsigned c1 = thr | (1u << shift), c2 = thr | (2u << shift), c3 = thr | (3u << shift);
            long long c[3] = {0, 0, 0};
            smp_for_each(vals, V, [&](int, float v) { unsigned k = xr_key(v); c[0] += (k >= c1); c[1] += (k >= c2); c[2] += (k >= c3); });
            blk_sum3_ll(c, sh);
            // at least k keys are >= a candidate: the k-th largest is >= it
            thr = c[2] >= top_k ? c3 : (c[1] >= top_k ? c2 : (c[0] >= top_k ? c1 : thr));
        }
        long long gt = 0;
        smp_for_each(vals, V, [&](int, float v) { gt += (xr_key(v) > thr); });
        gt = blk_sum_ll(gt, sh);
        cut.thr = thr; cut.n_eq = (long long)top_k - gt;      // that many of the equal keys, by id
    }
    // id bound for equal keys (V when all of them survive)
    int eq_id_end = V;
    if (cut.n_eq >= 0) {
        long long eq = 0;
        smp_for_each(vals, V, [&](int, float v) { eq += (xr_key(v) == cut.thr); });
        eq = blk_sum_ll(eq, sh);
        if (cut.n_eq < eq) eq_id_end = nth_equal_id(V, vals, cut.thr, cut.n_eq, sh);
    }
#define SURVIVES(i, k) ((k) > cut.thr || ((k) == cut.thr && (i) < eq_id_end))

    // ---- mass of the survivors ----
    double Z = 0.0;
    smp_for_each(vals, V, [&](int i, float v) { unsigned k = xr_key(v); if (SURVIVES(i, k)) Z += (double)expf(v - mx); });
    Z = blk_sum_d(Z, sh);

    // ---- top-p: shortest prefix with cumulative probability >= top_p ----
    float top_p = a.top_p[row];
    if (top_p < 1.0f) {
        double target = (double)top_p * Z;
        // largest key x with mass{key >= x} >= target
        unsigned thr = 0;
        for (int shift = 30; shift >= 0; shift -= 2) {
            const unsigned c1 = thr | (1u << shift), c2 = thr | (2u << shift), c3 = thr | (3u << shift);
            double ms[3] = {0.0, 0.0, 0.0};
            smp_for_each(vals, V, [&](int i, float v) {
                unsigned k = xr_key(v);
                if (k >= c1 && SURVIVES(i, k)) {
                    double e = (double)expf(v - mx);
                    ms[0] += e; ms[1] += k >= c2 ? e : 0.0; ms[2] += k >= c3 ? e : 0.0;
                }
            });
            blk_sum3_d(ms, sh);
            thr = ms[2] >= target ? c3 : (ms[1] >= target ? c2 : (ms[0] >= target ? c1 : thr));
        }
        {
            // among equal keys at thr, keep only as many (by id) as the prefix needs; if thr is also where top-k cut,
            // no more than top-k left there
            double gtm = 0.0; long long eqn = 0;
            smp_for_each(vals, V, [&](int, float v) { unsigned k = xr_key(v); if (k > thr) gtm += (double)expf(v - mx); eqn += (k == thr); });
            gtm = blk_sum_d(gtm, sh);
            eqn = blk_sum_ll(eqn, sh);
            long long avail = (thr == cut.thr && cut.n_eq >= 0 && cut.n_eq < eqn) ? cut.n_eq : eqn;
            long long need = avail;
            if (avail > 1) {
                // each equal candidate adds e; the prefix ends at the first whose cumulative sum reaches target
                float vt = __uint_as_float((thr & 0x80000000u) ? (thr & 0x7fffffffu) : ~thr);
                double e = (double)expf(vt - mx);
                long long c = (long long)ceil((target - gtm) / e - 1e-9);
                if (c < 1) c = 1;
                if (c < need) need = c;
            }
            cut.thr = thr; cut.n_eq = need;
            eq_id_end = need < eqn ? nth_equal_id(V, vals, thr, need, sh) : V;
        }
        Z = 0.0;
        smp_for_each(vals, V, [&](int i, float v) { unsigned k = xr_key(v); if (SURVIVES(i, k)) Z += (double)expf(v - mx); });
        Z = blk_sum_d(Z, sh);
    }

    // ---- min-p: drop candidates with p < min_p * p_max; the best candidate has exp(v - mx) = 1 ----
    float min_p = a.min_p[row];
    float e_floor = min_p > 0.f ? min_p : 0.f;
    if (e_floor > 0.f) {
        Z = 0.0;
        smp_for_each(vals, V, [&](int i, float v) {
            unsigned k = xr_key(v); float e = expf(v - mx);
            if (SURVIVES(i, k) && e >= e_floor) Z += (double)e;
        });
        Z = blk_sum_d(Z, sh);
    }
#define FINAL(i, k, e) (SURVIVES(i, k) && (e) >= e_floor)

    // ---- the pick: first candidate whose cumulative mass exceeds r * Z ----
    double want = (double)a.draw[row] * Z;
    unsigned thr = 0; bool any = false;
    for (int shift = 30; shift >= 0; shift -= 2) {
        const unsigned c1 = thr | (1u << shift), c2 = thr | (2u << shift), c3 = thr | (3u << shift);
        double ms[3] = {0.0, 0.0, 0.0};
        smp_for_each(vals, V, [&](int i, float v) {
            unsigned k = xr_key(v);
            if (k >= c1) {
                float e = expf(v - mx);
                if (FINAL(i, k, e)) { ms[0] += (double)e; ms[1] += k >= c2 ? (double)e : 0.0; ms[2] += k >= c3 ? (double)e : 0.0; }
            }
        });
        blk_sum3_d(ms, sh);
        if (ms[2] > want) { thr = c3; any = true; }
        else if (ms[1] > want) { thr = c2; any = true; }
        else if (ms[0] > want) { thr = c1; any = true; }
    }
    // candidates with key == thr that are in the final set, and the mass above them
    double gtm = 0.0; long long eqn = 0;
    smp_for_each(vals, V, [&](int i, float v) {
        unsigned k = xr_key(v); float e = expf(v - mx);
        if (FINAL(i, k, e)) { if (k > thr) gtm += (double)e; else if (k == thr) eqn++; }
    });
    gtm = blk_sum_d(gtm, sh);
    eqn = blk_sum_ll(eqn, sh);
    int pick;
    if (!any || eqn == 0) {
        // the walk ran off the end (r * Z rounded up to the whole mass): the reference returns the last
        // candidate (src/sample.c:119); that is the smallest final key, largest id
        unsigned lowk = 0xffffffffu; int lowi = -1;
        for (int i = tid; i < V; i += SMP_THREADS) {
            unsigned k = xr_key(vals[i]); float e = expf(vals[i] - mx);
            if (FINAL(i, k, e) && (k < lowk || (k == lowk && i > lowi))) { lowk = k; lowi = i; }
        }
        __syncthreads();
        unsigned* ks = (unsigned*)sh; int* is = (int*)(sh + 520);
        ks[tid] = lowk; is[tid] = lowi;
        __syncthreads();
        if (tid == 0) {
            for (int t = 1; t < SMP_THREADS; t++) if (is[t] >= 0 && (ks[t] < lowk || (ks[t] == lowk && is[t] > lowi) || lowi < 0)) { lowk = ks[t]; lowi = is[t]; }
            a.out[row] = lowi < 0 ? 0 : lowi;
        }
        return;
    }
    long long nth = 0;
    if (eqn > 1) {
        float vt = __uint_as_float((thr & 0x80000000u) ? (thr & 0x7fffffffu) : ~thr);
        double e = (double)expf(vt - mx);
        nth = (long long)floor((want - gtm) / e);
        if (nth < 0) nth = 0;
        if (nth >= eqn) nth = eqn - 1;
    }
    pick = nth_equal_id(V, vals, thr, nth, sh);
    if (tid == 0) a.out[row] = pick;
}

// ---------------------------------------------------------------------------------------------
// The same chain with a row spread over a cluster of SMP_CL blocks.  One block re-reads its row from L2 for
// every pass of a descent (some sixty passes of half a megabyte at what one SM can load); here every thread keeps
// SMP_PER consecutive values of the row in registers, a pass is arithmetic on those, a block-wide sum, and one
// exchange of the blocks' sums through distributed shared memory.  All blocks of a cluster add the same numbers
// in the same order (blocks in rank order), so they take the same decisions, and whatever guards an exchange is
// a function of such sums and of the row's parameters only: the blocks of a cluster always meet at the same
// barriers.  Vocabularies above SMP_CL * SMP_THREADS * SMP_PER keep the one-block kernel.
// ---------------------------------------------------------------------------------------------
#define SMP_CL 8
#define SMP_PER 16

struct SmpCluster {
    unsigned long long (*slots)[SMP_CL][3];     // shared memory [2][SMP_CL][3]: what each block sent, by exchange parity
    double* sh;                                  // the block sums' scratch
    int phase, rank;
};

// Every thread of the block holds the same three words; afterwards smp_cl_get(c, r, j) is word j of block r.
// Two sets of slots alternate: a block can be one exchange ahead of another, never two (the barrier), so what it
// writes is never what the other still reads.
__device__ __forceinline__ void smp_cl_exchange(SmpCluster& c, unsigned long long w0, unsigned long long w1, unsigned long long w2) {
    if (threadIdx.x < SMP_CL) {
        uint32_t local = (uint32_t)__cvta_generic_to_shared(&c.slots[c.phase][c.rank][0]), remote;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"((uint32_t)threadIdx.x));
        asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(remote), "l"(w0) : "memory");
        asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(remote + 8), "l"(w1) : "memory");
        asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(remote + 16), "l"(w2) : "memory");
    }
    __syncwarp();
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    c.phase ^= 1;
}
__device__ __forceinline__ unsigned long long smp_cl_get(const SmpCluster& c, int r, int j) { return c.slots[c.phase ^ 1][r][j]; }

__device__ __forceinline__ void smp_cl_sum3_ll(SmpCluster& c, long long (&v)[3]) {
    blk_sum3_ll(v, c.sh);
    smp_cl_exchange(c, (unsigned long long)v[0], (unsigned long long)v[1], (unsigned long long)v[2]);
#pragma unroll
    for (int j = 0; j < 3; j++) {
        long long t = 0;
        for (int r = 0; r < SMP_CL; r++) t += (long long)smp_cl_get(c, r, j);
        v[j] = t;
    }
}
__device__ __forceinline__ void smp_cl_sum3_d(SmpCluster& c, double (&v)[3]) {
    blk_sum3_d(v, c.sh);
    smp_cl_exchange(c, (unsigned long long)__double_as_longlong(v[0]), (unsigned long long)__double_as_longlong(v[1]),
                    (unsigned long long)__double_as_longlong(v[2]));
#pragma unroll
    for (int j = 0; j < 3; j++) {
        double t = 0.0;
        for (int r = 0; r < SMP_CL; r++) t += __longlong_as_double((long long)smp_cl_get(c, r, j));
        v[j] = t;
    }
}
__device__ __forceinline__ double smp_cl_sum_d(SmpCluster& c, double x) { double v[3] = {x, 0.0, 0.0}; smp_cl_sum3_d(c, v); return v[0]; }
__device__ __forceinline__ long long smp_cl_sum_ll(SmpCluster& c, long long x) { long long v[3] = {x, 0, 0}; smp_cl_sum3_ll(c, v); return v[0]; }

// One exchange for a sum of doubles and a count.
__device__ __forceinline__ void smp_cl_sum_d_ll(SmpCluster& c, double& d, long long& n) {
    d = blk_sum_d(d, c.sh);
    n = blk_sum_ll(n, c.sh);
    smp_cl_exchange(c, (unsigned long long)__double_as_longlong(d), (unsigned long long)n, 0ull);
    double td = 0.0; long long tn = 0;
    for (int r = 0; r < SMP_CL; r++) { td += __longlong_as_double((long long)smp_cl_get(c, r, 0)); tn += (long long)smp_cl_get(c, r, 1); }
    d = td; n = tn;
}

// id such that exactly `n` candidates with key == thr have an id below it.  A thread's ids are consecutive and
// threads, then blocks, follow one another in id order, so a prefix over (block, thread) is a prefix over ids.
template <int PER>
__device__ int smp_cl_nth_equal_id(SmpCluster& c, int V, const float (&v)[PER], int base, int nvalid, unsigned thr, long long n) {
    long long mine = 0;
#pragma unroll
    for (int j = 0; j < PER; j++) mine += (j < nvalid && xr_key(v[j]) == thr);
    long long* s = (long long*)c.sh + 40;
    __shared__ int found, owner;
    __shared__ long long owner_skip;
    __syncthreads();
    s[threadIdx.x] = mine;
    if (threadIdx.x == 0) { found = V; owner = -1; }
    const long long total = blk_sum_ll(mine, c.sh);              // (its barriers also publish s[] and found)
    smp_cl_exchange(c, (unsigned long long)total, 0ull, 0ull);
    long long before = 0;
    for (int r = 0; r < c.rank; r++) before += (long long)smp_cl_get(c, r, 0);
    const long long local = n - before;                           // the wanted one is this block's local-th, if it is here
    if (threadIdx.x == 0 && local >= 0 && local < total) {
        long long run = 0;
        for (int t = 0; t < SMP_THREADS; t++) {
            if (run + s[t] > local) { owner = t; owner_skip = local - run; break; }
            run += s[t];
        }
    }
    __syncthreads();
    if ((int)threadIdx.x == owner) {
        long long cnt = 0;
#pragma unroll
        for (int j = 0; j < PER; j++)
            if (j < nvalid && xr_key(v[j]) == thr) { if (cnt == owner_skip) found = base + j; cnt++; }
    }
    __syncthreads();
    smp_cl_exchange(c, (unsigned long long)found, 0ull, 0ull);
    int f = V;
    for (int r = 0; r < SMP_CL; r++) f = min(f, (int)smp_cl_get(c, r, 0));
    __syncthreads();                                              // found and owner may be written again by the next call
    return f;
}

template <int PER>
__global__ void __launch_bounds__(SMP_THREADS)
k_sample_cluster(SampleArgs a) {
    xr_pdl_launch();
    __shared__ double sh[40 + SMP_THREADS];
    __shared__ float sh_f[33];
    __shared__ int sh_i[33];
    __shared__ unsigned long long slots[2][SMP_CL][3];
    __shared__ int rec_tok[SMP_RECENT], rec_cnt[SMP_RECENT];
    const int row = blockIdx.x / SMP_CL, tid = threadIdx.x;
    SmpCluster c{slots, sh, 0, (int)(blockIdx.x % SMP_CL)};
    const float* lg = a.logits + (size_t)row * a.ld;
    // (the rows' parameters are written before the step's kernels are queued: they may be read before the wait)
    const float temp = a.temp[row];
    const int V = a.V;
    xr_pdl_wait();
    if (a.todo != nullptr && a.todo[(size_t)row * a.todo_stride] == 0) return;      // (the whole cluster: nobody writes these words here)
    if (temp <= 0.f) {                              // a greedy row: one block does it (the whole cluster leaves here)
        if (c.rank == 0) smp_argmax(lg, V, a.out + row, sh_f, sh_i);
        return;
    }
    // "this block runs": nobody writes into a block's shared memory before all of the cluster have begun
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");

    // ---- the thread's values: ids base .. base + nvalid - 1 ----
    const int base = (c.rank * SMP_THREADS + tid) * PER;
    const int nvalid = V - base < 0 ? 0 : (V - base < PER ? V - base : PER);
    float v[PER];
    if (nvalid == PER && ((((uintptr_t)(lg + base)) & 15) == 0)) {
        const float4* src = reinterpret_cast<const float4*>(lg + base);
        float4 q[PER / 4];
#pragma unroll
        for (int k = 0; k < PER / 4; k++) q[k] = xr_ld_now4(src + k);
#pragma unroll
        for (int k = 0; k < PER / 4; k++) { xr_ld_fence(q[k]); v[4 * k] = q[k].x; v[4 * k + 1] = q[k].y; v[4 * k + 2] = q[k].z; v[4 * k + 3] = q[k].w; }
    } else {
#pragma unroll
        for (int j = 0; j < PER; j++) v[j] = j < nvalid ? lg[base + j] : -INFINITY;
    }
    // ---- repeat penalty, once per occurrence in the window (src/sample.c:148-166) ----
    const float pen = a.penalty[row];
    if (a.recent != nullptr && pen != 1.0f) {
        if (tid < SMP_RECENT) rec_tok[tid] = smp_window_entry(a, row, tid);
        __syncthreads();
        int mine = -1, cnt = 0;
        if (tid < SMP_RECENT) {
            const int tok = rec_tok[tid];
            bool first = tok >= 0 && tok < V;
            if (first)
                for (int j = 0; j < SMP_RECENT; j++) { if (rec_tok[j] == tok) { cnt++; if (j < tid) first = false; } }
            mine = first ? tok : -1;
        }
        __syncthreads();
        if (tid < SMP_RECENT) { rec_tok[tid] = mine; rec_cnt[tid] = cnt; }
        __syncthreads();
        for (int e = 0; e < SMP_RECENT; e++) {
            const int off = rec_tok[e] - base;
            if (off >= 0 && off < nvalid) {
#pragma unroll
                for (int j = 0; j < PER; j++)
                    if (j == off) { float x = v[j]; for (int k = 0; k < rec_cnt[e]; k++) x = x > 0.f ? x / pen : x * pen; v[j] = x; }
            }
        }
    }
    // ---- scale, and the row's maximum ----
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < PER; j++) { v[j] = v[j] / temp; if (j < nvalid) mx = fmaxf(mx, v[j]); }
    mx = xr_warp_max(mx);
    __syncthreads();
    if ((tid & 31) == 0) sh_f[tid >> 5] = mx;
    __syncthreads();
    if (tid < 32) { float t = sh_f[tid]; t = xr_warp_max(t); if (tid == 0) sh_f[32] = t; }
    __syncthreads();
    smp_cl_exchange(c, (unsigned long long)__float_as_uint(sh_f[32]), 0ull, 0ull);
    mx = -INFINITY;
    for (int r = 0; r < SMP_CL; r++) mx = fmaxf(mx, __uint_as_float((unsigned)smp_cl_get(c, r, 0)));

    Cut cut{0u, -1};               // everything survives
    const int top_k = a.top_k[row];
    // ---- top-k: the k-th largest key by descending over the key bits with counts ----
    if (top_k > 0 && top_k < V) {
        unsigned thr = 0;
        for (int shift = 30; shift >= 0; shift -= 2) {
            const unsigned c1 = thr | (1u << shift), c2 = thr | (2u << shift), c3 = thr | (3u << shift);
            long long n[3] = {0, 0, 0};
#pragma unroll
            for (int j = 0; j < PER; j++)
                if (j < nvalid) { unsigned k = xr_key(v[j]); n[0] += (k >= c1); n[1] += (k >= c2); n[2] += (k >= c3); }
            smp_cl_sum3_ll(c, n);
            thr = n[2] >= top_k ? c3 : (n[1] >= top_k ? c2 : (n[0] >= top_k ? c1 : thr));
        }
        long long gt = 0;
#pragma unroll
        for (int j = 0; j < PER; j++) gt += (j < nvalid && xr_key(v[j]) > thr);
        gt = smp_cl_sum_ll(c, gt);
        cut.thr = thr; cut.n_eq = (long long)top_k - gt;      // that many of the equal keys, by id
    }
    // id bound for equal keys (V when all of them survive)
    int eq_id_end = V;
    if (cut.n_eq >= 0) {
        long long eq = 0;
#pragma unroll
        for (int j = 0; j < PER; j++) eq += (j < nvalid && xr_key(v[j]) == cut.thr);
        eq = smp_cl_sum_ll(c, eq);
        if (cut.n_eq < eq) eq_id_end = smp_cl_nth_equal_id<PER>(c, V, v, base, nvalid, cut.thr, cut.n_eq);
    }
#define CL_SURVIVES(i, k) ((k) > cut.thr || ((k) == cut.thr && (i) < eq_id_end))

    // ---- mass of the survivors ----
    double Z = 0.0;
#pragma unroll
    for (int j = 0; j < PER; j++)
        if (j < nvalid) { unsigned k = xr_key(v[j]); if (CL_SURVIVES(base + j, k)) Z += (double)expf(v[j] - mx); }
    Z = smp_cl_sum_d(c, Z);

    // ---- top-p: shortest prefix with cumulative probability >= top_p ----
    const float top_p = a.top_p[row];
    if (top_p < 1.0f) {
        const double target = (double)top_p * Z;
        unsigned thr = 0;                       // largest key x with mass{key >= x} >= target
        for (int shift = 30; shift >= 0; shift -= 2) {
            const unsigned c1 = thr | (1u << shift), c2 = thr | (2u << shift), c3 = thr | (3u << shift);
            double ms[3] = {0.0, 0.0, 0.0};
#pragma unroll
            for (int j = 0; j < PER; j++) {
                unsigned k = xr_key(v[j]);
                if (j < nvalid && k >= c1 && CL_SURVIVES(base + j, k)) {
                    double e = (double)expf(v[j] - mx);
                    ms[0] += e; ms[1] += k >= c2 ? e : 0.0; ms[2] += k >= c3 ? e : 0.0;
                }
            }
            smp_cl_sum3_d(c, ms);
            thr = ms[2] >= target ? c3 : (ms[1] >= target ? c2 : (ms[0] >= target ? c1 : thr));
        }
        // among equal keys at thr, keep only as many (by id) as the prefix needs; if thr is also where top-k cut,
        // no more than top-k left there
        double gtm = 0.0; long long eqn = 0;
#pragma unroll
        for (int j = 0; j < PER; j++)
            if (j < nvalid) { unsigned k = xr_key(v[j]); if (k > thr) gtm += (double)expf(v[j] - mx); eqn += (k == thr); }
        smp_cl_sum_d_ll(c, gtm, eqn);
        const long long avail = (thr == cut.thr && cut.n_eq >= 0 && cut.n_eq < eqn) ? cut.n_eq : eqn;
        long long need = avail;
        if (avail > 1) {
            // each equal candidate adds e; the prefix ends at the first whose cumulative sum reaches target
            float vt = __uint_as_float((thr & 0x80000000u) ? (thr & 0x7fffffffu) : ~thr);
            double e = (double)expf(vt - mx);
            long long n = (long long)ceil((target - gtm) / e - 1e-9);
            if (n < 1) n = 1;
            if (n < need) need = n;
        }
        cut.thr = thr; cut.n_eq = need;
        eq_id_end = need < eqn ? smp_cl_nth_equal_id<PER>(c, V, v, base, nvalid, thr, need) : V;
        Z = 0.0;
#pragma unroll
        for (int j = 0; j < PER; j++)
            if (j < nvalid) { unsigned k = xr_key(v[j]); if (CL_SURVIVES(base + j, k)) Z += (double)expf(v[j] - mx); }
        Z = smp_cl_sum_d(c, Z);
    }

    // ---- min-p: drop candidates with p < min_p * p_max; the best candidate has exp(v - mx) = 1 ----
    const float min_p = a.min_p[row];
    const float e_floor = min_p > 0.f ? min_p : 0.f;
    if (e_floor > 0.f) {
        Z = 0.0;
#pragma unroll
        for (int j = 0; j < PER; j++)
            if (j < nvalid) { unsigned k = xr_key(v[j]); float e = expf(v[j] - mx); if (CL_SURVIVES(base + j, k) && e >= e_floor) Z += (double)e; }
        Z = smp_cl_sum_d(c, Z);
    }
#define CL_FINAL(i, k, e) (CL_SURVIVES(i, k) && (e) >= e_floor)

    // ---- the pick: first candidate whose cumulative mass exceeds r * Z ----
    const double want = (double)a.draw[row] * Z;
    unsigned thr = 0; bool any = false;
    for (int shift = 30; shift >= 0; shift -= 2) {
        const unsigned c1 = thr | (1u << shift), c2 = thr | (2u << shift), c3 = thr | (3u << shift);
        double ms[3] = {0.0, 0.0, 0.0};
#pragma unroll
        for (int j = 0; j < PER; j++) {
            unsigned k = xr_key(v[j]);
            if (j < nvalid && k >= c1) {
                float e = expf(v[j] - mx);
                if (CL_FINAL(base + j, k, e)) { ms[0] += (double)e; ms[1] += k >= c2 ? (double)e : 0.0; ms[2] += k >= c3 ? (double)e : 0.0; }
            }
        }
        smp_cl_sum3_d(c, ms);
        if (ms[2] > want) { thr = c3; any = true; }
        else if (ms[1] > want) { thr = c2; any = true; }
        else if (ms[0] > want) { thr = c1; any = true; }
    }
    // candidates with key == thr that are in the final set, and the mass above them
    double gtm = 0.0; long long eqn = 0;
#pragma unroll
    for (int j = 0; j < PER; j++)
        if (j < nvalid) {
            unsigned k = xr_key(v[j]); float e = expf(v[j] - mx);
            if (CL_FINAL(base + j, k, e)) { if (k > thr) gtm += (double)e; else if (k == thr) eqn++; }
        }
    smp_cl_sum_d_ll(c, gtm, eqn);
    if (!any || eqn == 0) {
        // the walk ran off the end (r * Z rounded up to the whole mass): the reference returns the last
        // candidate (src/sample.c:119); that is the smallest final key, largest id.  Both in one word whose
        // minimum is wanted: key above, inverted id below.
        unsigned long long low = ~0ull;
#pragma unroll
        for (int j = 0; j < PER; j++)
            if (j < nvalid) {
                unsigned k = xr_key(v[j]); float e = expf(v[j] - mx);
                if (CL_FINAL(base + j, k, e)) {
                    unsigned long long w = ((unsigned long long)k << 32) | (unsigned long long)(0xffffffffu - (unsigned)(base + j));
                    low = w < low ? w : low;
                }
            }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) { unsigned long long t = __shfl_xor_sync(0xffffffffu, low, o); low = t < low ? t : low; }
        unsigned long long* ws = (unsigned long long*)sh;
        __syncthreads();
        if ((tid & 31) == 0) ws[tid >> 5] = low;
        __syncthreads();
        low = ws[0];
        for (int w = 1; w < SMP_THREADS / 32; w++) low = ws[w] < low ? ws[w] : low;
        smp_cl_exchange(c, low, 0ull, 0ull);
        for (int r = 0; r < SMP_CL; r++) { unsigned long long t = smp_cl_get(c, r, 0); low = t < low ? t : low; }
        if (c.rank == 0 && tid == 0) a.out[row] = low == ~0ull ? 0 : (int)(0xffffffffu - (unsigned)(low & 0xffffffffull));
        return;
    }
    long long nth = 0;
    if (eqn > 1) {
        float vt = __uint_as_float((thr & 0x80000000u) ? (thr & 0x7fffffffu) : ~thr);
        double e = (double)expf(vt - mx);
        nth = (long long)floor((want - gtm) / e);
        if (nth < 0) nth = 0;
        if (nth >= eqn) nth = eqn - 1;
    }
    const int pick = smp_cl_nth_equal_id<PER>(c, V, v, base, nvalid, thr, nth);
    if (c.rank == 0 && tid == 0) a.out[row] = pick;
#undef CL_SURVIVES
#undef CL_FINAL
}

static int launch_sample_cluster(const SampleArgs& a, int rows, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(rows * SMP_CL); cfg.blockDim = dim3(SMP_THREADS); cfg.dynamicSmemBytes = 0; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = SMP_CL; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = xr_pdl_enabled() ? 2 : 1;
    cudaLaunchKernelEx(&cfg, k_sample_cluster<SMP_PER>, a);
    return xr_launch_status();
}

// Whether these rows go to the cluster kernel (xr_sample_one_block is the entry point of the other).  A cluster
// block fills an SM (1,024 threads of 64 registers), so clusters run in waves of (SMs / 8) rows.  Measured at a
// vocabulary of 128,256 with top-k and top-p: 180 us a wave (8 rows 180, 24 rows 355, 48 rows 700), where the
// one-block kernel takes 715 us for any number of rows up to the SM count; up to two waves the cluster kernel wins.
static bool smp_use_cluster(int rows, int V) {
    int sms = xr_sm_count();
    if (sms < SMP_CL) sms = SMP_CL;
    if (V <= SMP_THREADS || (long long)V > (long long)SMP_CL * SMP_THREADS * SMP_PER) return false;
    return rows <= 2 * (sms / SMP_CL);
}

// ---------------------------------------------------------------------------------------------
// Teacher-forced scoring: out[row] = log P(target[row]) under softmax(logits[row]), the arithmetic of the
// reference's --score mode (src/main.c:1395-1405): float maximum, sum of expf(v - max) in double, float result
// v[target] - (max + logf((float)sum)).  One block a row.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(SMP_THREADS)
k_logprob(const float* logits, long long ld, int V, const int* target, float* out) {
    xr_pdl_launch();
    __shared__ double sh[40 + 64];
    __shared__ float sh_f[33];
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* lg = logits + (size_t)row * ld;
    xr_pdl_wait();
    float mx = -INFINITY;
    smp_for_each(lg, V, [&](int, float v) { mx = fmaxf(mx, v); });
    mx = xr_warp_max(mx);
    if ((tid & 31) == 0) sh_f[tid >> 5] = mx;
    __syncthreads();
    if (tid < 32) { float t = sh_f[tid]; t = xr_warp_max(t); if (tid == 0) sh_f[32] = t; }
    __syncthreads();
    mx = sh_f[32];
    double sum = 0.0;
    smp_for_each(lg, V, [&](int, float v) { sum += (double)expf(v - mx); });
    sum = blk_sum_d(sum, sh);
    if (tid == 0) {
        int t = target[row];
        out[row] = (t >= 0 && t < V) ? lg[t] - (mx + logf((float)sum)) : -INFINITY;
    }
}

XR_EXPORT int xr_logprob(const float* logits, long long ld, int rows, int V, const int* target, float* out, cudaStream_t stream) {
    if (rows < 1 || V < 1 || ld < V) return XR_ERR_ARG;
    xr_launch(k_logprob, dim3(rows), dim3(SMP_THREADS), 0, stream, logits, ld, V, target, out);
    return xr_launch_status();
}

// scratch: [rows, V] floats when any row has temp > 0 (may be null when all rows are greedy).
static int launch_sample_block(const SampleArgs& a, int rows, float* scratch, int shortcuts, cudaStream_t stream) {
    // candidates (keys, ids, values in order, ids in order) and one bit per token id for the window of recent tokens
    constexpr int DYN_MAX = SMP_DYN_MAX;
    const long long dyn = (long long)SMP_CAP * 16 + ((long long)(a.V + 31) / 32) * 4;
    if (shortcuts && dyn > DYN_MAX) return XR_ERR_ARG;              // (a vocabulary of more than 786,432; xr_sample checks before)
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(k_sample, cudaFuncAttributeMaxDynamicSharedMemorySize, DYN_MAX) != cudaSuccess) return XR_ERR_LAUNCH;
        configured = true;
    }
    xr_launch(k_sample, dim3(rows), dim3(SMP_THREADS), shortcuts ? (size_t)dyn : 0, stream, a, scratch, shortcuts ? 1 : 0);
    return xr_launch_status();
}

// shortcuts: take the reference's short cuts (one block a row); 0: the threshold descents only, a cluster of eight
// blocks a row when the rows are few.
XR_EXPORT int xr_sample(const float* logits, long long ld, int rows, int V, const float* temp, const int* top_k,
                        const float* top_p, const float* min_p, const float* penalty, const float* draw,
                        const int* recent, float* scratch, int* out, int shortcuts, const int* pending, const int* feed,
                        const int* exempt, cudaStream_t stream) {
    if (rows < 1 || V < 1 || ld < V) return XR_ERR_ARG;
    if (pending != nullptr && (feed == nullptr || exempt == nullptr || recent == nullptr)) return XR_ERR_ARG;
    SampleArgs a{logits, ld, V, temp, top_k, top_p, min_p, penalty, draw, recent, out, pending, feed, exempt, nullptr, 0};
    if ((long long)SMP_CAP * 16 + ((long long)(V + 31) / 32) * 4 > SMP_DYN_MAX) shortcuts = 0;      // (more than 786,432 values a row)
    if (shortcuts) {
        // the short cuts for every row, then the long way for the rows they left open (usually none: the second launch
        // then reads one word a row and ends).  The words lie at the start of each row's staging area.
        if (scratch == nullptr) return XR_ERR_ARG;
        a.todo = (const int*)scratch; a.todo_stride = V;
        int rc = launch_sample_block(a, rows, scratch, 1, stream);
        if (rc != XR_OK) return rc;
    }
    if (smp_use_cluster(rows, V)) return launch_sample_cluster(a, rows, stream);
    return launch_sample_block(a, rows, scratch, 0, stream);
}

// The one-block kernel whatever the width (what xr_sample falls back to; tests compare the two).
XR_EXPORT int xr_sample_one_block(const float* logits, long long ld, int rows, int V, const float* temp, const int* top_k,
                                  const float* top_p, const float* min_p, const float* penalty, const float* draw,
                                  const int* recent, float* scratch, int* out, cudaStream_t stream) {
    if (rows < 1 || V < 1 || ld < V) return XR_ERR_ARG;
    SampleArgs a{logits, ld, V, temp, top_k, top_p, min_p, penalty, draw, recent, out, nullptr, nullptr, nullptr, nullptr, 0};
    return launch_sample_block(a, rows, scratch, 0, stream);
}
