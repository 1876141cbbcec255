// Seeded normal values whose bits do not depend on the machine that draws them.
//
// out[i] = mean + std * z_i, where z_i is a function of (key, first + i) alone: a counter-based generator, so a
// tensor can be drawn on the device, on the CPU, whole or in pieces, and holds the same bits every time.  The
// same function is written with numpy in weights/random_fill.py; the two agree bit for bit because every step
// is either integer arithmetic or ONE correctly rounded float32 operation (add, multiply, divide, square
// root; never a fused multiply-add, never a library logarithm or cosine, whose last bits differ between
// implementations):
//
//   h      = mix64(key + (index + 1) * 0x9E3779B97F4A7C15)       (the splitmix64 finaliser)
//   u      = (2 * (h >> 41) + 1) * 2^-24                          in (0, 1), exact in float32
//   phase  = (h >> 8) & 0xFFFFFF                                  a 24-bit fraction of the full turn
//   z      = sqrt(-2 ln u) * cos(2 pi phase / 2^24)               (Box-Muller)
//
// ln u   : u = m * 2^e with m in (sqrt(1/2), sqrt(2)]; s = (m - 1) / (m + 1); ln m = 2 s (1 + s^2/3 + s^4/5 + s^6/7 + s^8/9)
// cosine : the top two bits of the phase pick the quadrant; the rest, centred, is x in [-pi/4, pi/4); sin x and
//          cos x by their series to x^9 and x^8; cos(x + pi/4) and sin(x + pi/4) from them; signs by quadrant.
//
// The reference's only generator is its fixture script's LCG (scripts/make-test-model.py:238-252): weights that
// anyone can re-make from a seed.  This is the same idea for tensors of any size on any device.
#include "common.cuh"

// constants: doubles rounded once to float32 (the numpy twin rounds the same doubles)
#define RF_SQRT2 ((float)1.4142135623730951)
#define RF_INV_SQRT2 ((float)0.7071067811865476)
#define RF_LN2 ((float)0.6931471805599453)
#define RF_QUARTER_STEP ((float)(1.5707963267948966 / 4194304.0))

__device__ __forceinline__ unsigned long long rf_mix64(unsigned long long z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}

// every float operation below is one IEEE operation, spelled out so that the compiler cannot fuse two of them
__device__ __forceinline__ float rf_horner(float p, float x, float c) { return __fadd_rn(__fmul_rn(p, x), c); }

__device__ __forceinline__ float rf_normal(unsigned long long key, unsigned long long index) {
    const unsigned long long h = rf_mix64(key + (index + 1ULL) * 0x9E3779B97F4A7C15ULL);
    // radius
    const unsigned int a = (unsigned int)(h >> 41);                 // 23 bits
    const float u = __fmul_rn((float)(int)(2u * a + 1u), (float)(1.0 / 16777216.0));      // * 2^-24, exact
    const unsigned int bits = __float_as_uint(u);
    int e = (int)(bits >> 23) - 127;
    float m = __uint_as_float((bits & 0x7FFFFFu) | 0x3F800000u);    // [1, 2)
    if (m > RF_SQRT2) { m = __fmul_rn(m, 0.5f); e += 1; }
    const float s = __fdiv_rn(__fadd_rn(m, -1.0f), __fadd_rn(m, 1.0f));
    const float s2 = __fmul_rn(s, s);
    float p = (float)(1.0 / 9.0);
    p = rf_horner(p, s2, (float)(1.0 / 7.0));
    p = rf_horner(p, s2, (float)(1.0 / 5.0));
    p = rf_horner(p, s2, (float)(1.0 / 3.0));
    p = rf_horner(p, s2, 1.0f);
    const float ln_m = __fmul_rn(__fmul_rn(2.0f, s), p);
    const float ln_u = __fadd_rn(__fmul_rn((float)e, RF_LN2), ln_m);
    const float r = __fsqrt_rn(__fmul_rn(-2.0f, ln_u));
    // angle
    const unsigned int b = (unsigned int)(h >> 8) & 0xFFFFFFu;
    const unsigned int q = b >> 22;
    const int w = (int)(b & 0x3FFFFFu) - (1 << 21);
    const float x = __fmul_rn((float)w, RF_QUARTER_STEP);           // * (pi/2) / 2^22
    const float x2 = __fmul_rn(x, x);
    float sp = (float)(1.0 / 362880.0);
    sp = rf_horner(sp, x2, (float)(-1.0 / 5040.0));
    sp = rf_horner(sp, x2, (float)(1.0 / 120.0));
    sp = rf_horner(sp, x2, (float)(-1.0 / 6.0));
    sp = rf_horner(sp, x2, 1.0f);
    const float sx = __fmul_rn(x, sp);
    float cp = (float)(1.0 / 40320.0);
    cp = rf_horner(cp, x2, (float)(-1.0 / 720.0));
    cp = rf_horner(cp, x2, (float)(1.0 / 24.0));
    cp = rf_horner(cp, x2, -0.5f);
    cp = rf_horner(cp, x2, 1.0f);
    const float s1 = __fmul_rn(__fadd_rn(sx, cp), RF_INV_SQRT2);    // sin(x + pi/4)
    const float c1 = __fmul_rn(__fadd_rn(cp, -sx), RF_INV_SQRT2);   // cos(x + pi/4)
    const float c = q == 0 ? c1 : (q == 1 ? -s1 : (q == 2 ? -c1 : s1));
    return __fmul_rn(r, c);
}

template <typename T>
__global__ void k_random_normal(T* out, long long n, unsigned long long key, unsigned long long first, float mean, float std) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = xr_from_f32<T>(__fadd_rn(mean, __fmul_rn(rf_normal(key, first + (unsigned long long)i), std)));
}

// out[i] = mean + std * z(key, first + i) for i in [0, n), rounded to `dtype` (bfloat16: nearest even).
XR_EXPORT int xr_random_normal(void* out, int dtype, long long n, unsigned long long key, unsigned long long first,
                               float mean, float std, cudaStream_t stream) {
    if (n < 0 || (dtype != XR_F32 && dtype != XR_BF16)) return XR_ERR_ARG;
    if (n == 0) return XR_OK;
    long long blocks = (n + 255) / 256;
    if (blocks > (long long)xr_sm_count() * 32) blocks = (long long)xr_sm_count() * 32;
    if (dtype == XR_F32) k_random_normal<float><<<(int)blocks, 256, 0, stream>>>((float*)out, n, key, first, mean, std);
    else k_random_normal<__nv_bfloat16><<<(int)blocks, 256, 0, stream>>>((__nv_bfloat16*)out, n, key, first, mean, std);
    return xr_launch_status();
}
