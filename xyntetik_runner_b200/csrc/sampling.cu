// Picking the next token from float32 logits on the device, one block per row.
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
// The reference sorts; this kernel never does.  Every cut above is a prefix of the same order, so it
// is described by a threshold in an order-preserving integer image of v (plus, among exact ties, a
// count of ids).  Thresholds are found by descending over the 32 key bits, each step one block-wide
// sum in a fixed order, which makes the result deterministic.
#include "common.cuh"
#include <math.h>

#define SMP_THREADS 1024
#define SMP_RECENT 256

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
};

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

__global__ void __launch_bounds__(SMP_THREADS)
k_sample(SampleArgs a, float* scratch /* [rows, V] scaled values, or null when nothing needs them */) {
    xr_pdl_launch();
    __shared__ double sh[40 + SMP_THREADS];
    __shared__ float sh_f[33];
    __shared__ int sh_i[33];
    int row = blockIdx.x, tid = threadIdx.x;
    const float* lg = a.logits + (size_t)row * a.ld;
    // (the rows' parameters are written before the step's kernels are queued: they may be read before the wait)
    float temp = a.temp[row];
    int V = a.V;
    xr_pdl_wait();

    if (temp <= 0.f) {
        // argmax, first index on ties (src/sample.c:169-172).  A row is half a megabyte that one block reads alone:
        // eight 16-byte loads a thread are issued as one run, so the row takes a few trips to L2, not dozens.
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
            if (tid == 0) a.out[row] = bi == 0x7fffffff ? 0 : bi;
        }
        return;
    }

    // Stage the row: copy, penalise the recent tokens (once per occurrence in the window, as the
    // reference's loop does, src/sample.c:148-166), then scale by 1/temp.  Later passes read the
    // staged values back, so every pass sees the same numbers.
    float* vals = scratch + (size_t)row * V;
    for (int i = tid; i < V; i += SMP_THREADS) vals[i] = lg[i];
    __syncthreads();
    float pen = a.penalty[row];
    if (a.recent != nullptr && pen != 1.0f && tid < SMP_RECENT) {
        const int* rec = a.recent + (size_t)row * SMP_RECENT;
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
    __syncthreads();
    float mx = -INFINITY;
    for (int i = tid; i < V; i += SMP_THREADS) {
        float v = vals[i] / temp;
        vals[i] = v;
        mx = fmaxf(mx, v);
    }
    mx = xr_warp_max(mx);
    if ((tid & 31) == 0) sh_f[tid >> 5] = mx;
    __syncthreads();
    if (tid < 32) { float t = sh_f[tid]; t = xr_warp_max(t); if (tid == 0) sh_f[32] = t; }
    __syncthreads();
    mx = sh_f[32];
    __syncthreads();

    Cut cut{0u, -1};               // everything survives
    int top_k = a.top_k[row];
    // ---- top-k: the k-th largest key by descending over the key bits with counts ----
    if (top_k > 0 && top_k < V) {
        unsigned thr = 0;
        for (int bit = 31; bit >= 0; bit--) {
            unsigned cand = thr | (1u << bit);
            long long c = 0;
            for (int i = tid; i < V; i += SMP_THREADS) c += (xr_key(vals[i]) >= cand);
            c = blk_sum_ll(c, sh);
            if (c >= top_k) thr = cand;       // at least k keys are >= cand: the k-th largest is >= cand
        }
        long long gt = 0;
        for (int i = tid; i < V; i += SMP_THREADS) gt += (xr_key(vals[i]) > thr);
        gt = blk_sum_ll(gt, sh);
        cut.thr = thr; cut.n_eq = (long long)top_k - gt;      // that many of the equal keys, by id
    }
    // id bound for equal keys (V when all of them survive)
    int eq_id_end = V;
    if (cut.n_eq >= 0) {
        long long eq = 0;
        for (int i = tid; i < V; i += SMP_THREADS) eq += (xr_key(vals[i]) == cut.thr);
        eq = blk_sum_ll(eq, sh);
        if (cut.n_eq < eq) eq_id_end = nth_equal_id(V, vals, cut.thr, cut.n_eq, sh);
    }
#define SURVIVES(i, k) ((k) > cut.thr || ((k) == cut.thr && (i) < eq_id_end))

    // ---- mass of the survivors ----
    double Z = 0.0;
    for (int i = tid; i < V; i += SMP_THREADS) { unsigned k = xr_key(vals[i]); if (SURVIVES(i, k)) Z += (double)expf(vals[i] - mx); }
    Z = blk_sum_d(Z, sh);

    // ---- top-p: shortest prefix with cumulative probability >= top_p ----
    float top_p = a.top_p[row];
    if (top_p < 1.0f) {
        double target = (double)top_p * Z;
        // largest key x with mass{key >= x} >= target
        unsigned thr = 0;
        for (int bit = 31; bit >= 0; bit--) {
            unsigned cand = thr | (1u << bit);
            double ms = 0.0;
            for (int i = tid; i < V; i += SMP_THREADS) { unsigned k = xr_key(vals[i]); if (k >= cand && SURVIVES(i, k)) ms += (double)expf(vals[i] - mx); }
            ms = blk_sum_d(ms, sh);
            if (ms >= target) thr = cand;
        }
        {
            // among equal keys at thr, keep only as many (by id) as the prefix needs; if thr is also where top-k cut,
            // no more than top-k left there
            double gtm = 0.0; long long eqn = 0;
            for (int i = tid; i < V; i += SMP_THREADS) { unsigned k = xr_key(vals[i]); if (k > thr) gtm += (double)expf(vals[i] - mx); eqn += (k == thr); }
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
        for (int i = tid; i < V; i += SMP_THREADS) { unsigned k = xr_key(vals[i]); if (SURVIVES(i, k)) Z += (double)expf(vals[i] - mx); }
        Z = blk_sum_d(Z, sh);
    }

    // ---- min-p: drop candidates with p < min_p * p_max; the best candidate has exp(v - mx) = 1 ----
    float min_p = a.min_p[row];
    float e_floor = min_p > 0.f ? min_p : 0.f;
    if (e_floor > 0.f) {
        Z = 0.0;
        for (int i = tid; i < V; i += SMP_THREADS) {
            unsigned k = xr_key(vals[i]); float e = expf(vals[i] - mx);
            if (SURVIVES(i, k) && e >= e_floor) Z += (double)e;
        }
        Z = blk_sum_d(Z, sh);
    }
#define FINAL(i, k, e) (SURVIVES(i, k) && (e) >= e_floor)

    // ---- the pick: first candidate whose cumulative mass exceeds r * Z ----
    double want = (double)a.draw[row] * Z;
    unsigned thr = 0; bool any = false;
    for (int bit = 31; bit >= 0; bit--) {
        unsigned cand = thr | (1u << bit);
        double ms = 0.0;
        for (int i = tid; i < V; i += SMP_THREADS) {
            unsigned k = xr_key(vals[i]); float e = expf(vals[i] - mx);
            if (k >= cand && FINAL(i, k, e)) ms += (double)e;
        }
        ms = blk_sum_d(ms, sh);
        if (ms > want) { thr = cand; any = true; }
    }
    // candidates with key == thr that are in the final set, and the mass above them
    double gtm = 0.0; long long eqn = 0;
    for (int i = tid; i < V; i += SMP_THREADS) {
        unsigned k = xr_key(vals[i]); float e = expf(vals[i] - mx);
        if (FINAL(i, k, e)) { if (k > thr) gtm += (double)e; else if (k == thr) eqn++; }
    }
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

// scratch: [rows, V] floats when any row has temp > 0 (may be null when all rows are greedy).
XR_EXPORT int xr_sample(const float* logits, long long ld, int rows, int V, const float* temp, const int* top_k,
                        const float* top_p, const float* min_p, const float* penalty, const float* draw,
                        const int* recent, float* scratch, int* out, cudaStream_t stream) {
    if (rows < 1 || V < 1 || ld < V) return XR_ERR_ARG;
    SampleArgs a{logits, ld, V, temp, top_k, top_p, min_p, penalty, draw, recent, out};
    xr_launch(k_sample, dim3(rows), dim3(SMP_THREADS), 0, stream, a, scratch);
    return xr_launch_status();
}
