// Random weights drawn on the device by a counter-based rule that the host restates operation for operation
// (ferrox_b200/weights/random_init.py), so that a tensor has the same bits wherever it is drawn and a model of
// any size can be checked against a plain implementation without going through a file.
//
//   element pair j of a tensor with key k:  x1 = mix(k + (2j+1) G), x2 = mix(k + (2j+2) G)   (64-bit, wrapping)
//   u = ((x >> 12) + 0.5) * 2^-52 in (0, 1);  r = sqrt(-2 ln u1);  element 2j = r cos(2 pi u2), 2j+1 = r sin(2 pi u2)
//   value = mean + std * element, rounded once to 32 bits and, for bfloat16, once more to nearest even.
//
// ln, cos and sin are evaluated here by series of additions, multiplications and divisions in 64-bit floating
// point, every one rounded by itself (the __d*_rn intrinsics are never contracted into fused multiply-adds), so the
// host's 64-bit arithmetic gives the same bits.  The reference's synthetic model is likewise one seeded generator
// for every tensor (crates/ferrox-models/src/decoder.rs:373-388).
#include "common.cuh"
#include "api.h"

namespace {

#define FX_RNG_GOLDEN 0x9E3779B97F4A7C15ull

__device__ __forceinline__ unsigned long long mix64(unsigned long long z)
{
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__device__ __forceinline__ double unit_open(unsigned long long x)
{
    // 52 random bits plus a half: exact in 64-bit floating point, never 0 or 1
    return __dmul_rn(__dadd_rn((double)(long long)(x >> 12), 0.5), 2.220446049250313e-16 /* 2^-52 */);
}

// ln u for u in (0, 1): u = m 2^e with m in [sqrt(1/2), sqrt(2)); ln m = 2 atanh(s), s = (m-1)/(m+1), by its series
// in s^2 (|s| < 0.172: eleven terms reach 1e-17); ln u = 2 s poly + e ln 2.
__device__ __forceinline__ double ln_exact_ops(double u)
{
    int e;
    double m = frexp(u, &e);                     // m in [0.5, 1), exact
    if (m < 0.7071067811865476) { m = __dmul_rn(m, 2.0); e -= 1; }
    const double s = __ddiv_rn(__dadd_rn(m, -1.0), __dadd_rn(m, 1.0));
    const double s2 = __dmul_rn(s, s);
    double p = __ddiv_rn(1.0, 21.0);
#pragma unroll
    for (int k = 9; k >= 0; --k) p = __dadd_rn(__dmul_rn(p, s2), __ddiv_rn(1.0, (double)(2 * k + 1)));
    return __dadd_rn(__dmul_rn(__dmul_rn(2.0, s), p), __dmul_rn((double)e, 0.6931471805599453));
}

// cos and sin of 2 pi u for u in (0, 1): the quarter turn k = floor(4u) and the rest f in [0, 1) are exact; the
// angle (pi/2) f is folded to at most pi/4 (f > 1/2: the complement, with cos and sin exchanged) and both series
// are summed to the tenth term (below 1e-18 there).
__device__ __forceinline__ void cos_sin_turn(double u, double& c_out, double& s_out)
{
    const double t = __dmul_rn(u, 4.0);
    const double kf = floor(t);
    const int k = (int)kf;
    double f = __dadd_rn(t, -kf);
    const bool fold = f > 0.5;
    if (fold) f = __dadd_rn(1.0, -f);
    const double a = __dmul_rn(f, 1.5707963267948966);
    const double a2 = __dmul_rn(a, a);
    // cos a = sum (-1)^n a^2n / (2n)!,  sin a = a sum (-1)^n a^2n / (2n+1)!   (Horner in a^2, n = 10 .. 0)
    double pc = 0.0, ps = 0.0;
#pragma unroll
    for (int n = 10; n >= 1; --n) {
        pc = __dmul_rn(__dadd_rn(1.0, -pc), __ddiv_rn(a2, (double)((2 * n - 1) * (2 * n))));
        ps = __dmul_rn(__dadd_rn(1.0, -ps), __ddiv_rn(a2, (double)((2 * n) * (2 * n + 1))));
    }
    double c = __dadd_rn(1.0, -pc);
    double s = __dmul_rn(a, __dadd_rn(1.0, -ps));
    if (fold) { const double x = c; c = s; s = x; }
    // quarter turns: (c, s) -> (-s, c) per turn
    switch (k & 3) {
        case 0: c_out = c; s_out = s; break;
        case 1: c_out = -s; s_out = c; break;
        case 2: c_out = -c; s_out = -s; break;
        default: c_out = s; s_out = -c; break;
    }
}

template <typename T>
__global__ void random_normal_kernel(T* __restrict__ out, long n, unsigned long long key, double mean, double stdev)
{
    const long n_pairs = (n + 1) >> 1;
    for (long j = blockIdx.x * (long)blockDim.x + threadIdx.x; j < n_pairs; j += (long)gridDim.x * blockDim.x) {
        const unsigned long long x1 = mix64(key + (2ull * (unsigned long long)j + 1ull) * FX_RNG_GOLDEN);
        const unsigned long long x2 = mix64(key + (2ull * (unsigned long long)j + 2ull) * FX_RNG_GOLDEN);
        const double r = __dsqrt_rn(__dmul_rn(-2.0, ln_exact_ops(unit_open(x1))));
        double c, s;
        cos_sin_turn(unit_open(x2), c, s);
        const double v0 = __dadd_rn(mean, __dmul_rn(stdev, __dmul_rn(r, c)));
        const double v1 = __dadd_rn(mean, __dmul_rn(stdev, __dmul_rn(r, s)));
        out[2 * j] = from_f32<T>(__double2float_rn(v0));
        if (2 * j + 1 < n) out[2 * j + 1] = from_f32<T>(__double2float_rn(v1));
    }
}

}  // namespace

// out[i] = mean + stdev * z_i for i < n, z the standard normal stream of `key`; dtype FX_F32 or FX_BF16.
extern "C" int fx_random_normal(void* out, int dtype, long n, unsigned long long key, double mean, double stdev,
                                void* stream)
{
    if (n <= 0) return FX_OK;
    if (dtype != FX_F32 && dtype != FX_BF16) return FX_ERR_DTYPE;
    const int threads = 256;
    const long pairs = (n + 1) / 2;
    const long cap = fx_sm_count() * 16L;
    const int blocks = (int)(fx_cdiv(pairs, threads) < cap ? fx_cdiv(pairs, threads) : cap);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == FX_F32) random_normal_kernel<float><<<blocks, threads, 0, st>>>((float*)out, n, key, mean, stdev);
    else random_normal_kernel<bf16><<<blocks, threads, 0, st>>>((bf16*)out, n, key, mean, stdev);
    return fx_launch_status();
}
