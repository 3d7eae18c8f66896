// The random-weights generator: element j of the tensor with key K is a pure function of (K, j),
// the same bits from the host (csrc/host/host.cpp), the device (csrc/fill.cu) and a NumPy twin in
// the tests.  Two splitmix64 outputs (the generator the reference's samplers use,
// crates/cli/src/flint.rs:318-325, device twin crates/cuda/kernels/common.cuh:113-119) give two
// 53-bit uniforms, Box-Muller a normal.  For the bits to agree everywhere no library logarithm
// or cosine is called: both are written out below in double precision with additions,
// multiplications, divisions and the square root only, each rounded on its own (the device code
// uses the _rn intrinsics, which the compiler never fuses; the host file is compiled with
// -ffp-contract=off).
#pragma once
#include <cstdint>
#include <cstring>

#if defined(__CUDACC__)
#define Q6K_HD __host__ __device__ __forceinline__
#else
#define Q6K_HD inline
#endif

namespace q6k_fill {

#if defined(__CUDA_ARCH__)
Q6K_HD double mul(double a, double b) { return __dmul_rn(a, b); }
Q6K_HD double add(double a, double b) { return __dadd_rn(a, b); }
Q6K_HD double quo(double a, double b) { return __ddiv_rn(a, b); }
Q6K_HD double root(double a) { return __dsqrt_rn(a); }
Q6K_HD float mulf(float a, float b) { return __fmul_rn(a, b); }
Q6K_HD float addf(float a, float b) { return __fadd_rn(a, b); }
#else
Q6K_HD double mul(double a, double b) { return a * b; }
Q6K_HD double add(double a, double b) { return a + b; }
Q6K_HD double quo(double a, double b) { return a / b; }
double sqrt_exact(double);          // IEEE square root: defined by the file that includes this on the host
Q6K_HD double root(double a) { return sqrt_exact(a); }
Q6K_HD float mulf(float a, float b) { return a * b; }
Q6K_HD float addf(float a, float b) { return a + b; }
#endif

Q6K_HD uint64_t mix(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}

Q6K_HD double from_bits(uint64_t b) {
    double d;
#if defined(__CUDA_ARCH__)
    d = __longlong_as_double((long long)b);
#else
    std::memcpy(&d, &b, sizeof d);
#endif
    return d;
}
Q6K_HD uint64_t to_bits(double d) {
#if defined(__CUDA_ARCH__)
    return (uint64_t)__double_as_longlong(d);
#else
    uint64_t b;
    std::memcpy(&b, &d, sizeof b);
    return b;
#endif
}

// ln(n * 2^-53) for an integer n in [1, 2^53]: n = m * 2^e with m in [sqrt(1/2), sqrt(2)], ln m = 2 atanh(s),
// s = (m - 1) / (m + 1), |s| <= 0.1716: eleven terms of the series reach 1e-17.
Q6K_HD double log_of_uniform(uint64_t n) {
    const uint64_t bits = to_bits((double)n);                    // exact: n <= 2^53
    int e = (int)((bits >> 52) & 0x7ff) - 1023;
    double m = from_bits((bits & 0x000FFFFFFFFFFFFFULL) | 0x3FF0000000000000ULL);      // [1, 2)
    if (m > 1.4142135623730951) {
        m = mul(m, 0.5);
        e += 1;
    }
    const double s = quo(add(m, -1.0), add(m, 1.0)), s2 = mul(s, s);
    double p = quo(1.0, 23.0);
    p = add(mul(p, s2), quo(1.0, 21.0));
    p = add(mul(p, s2), quo(1.0, 19.0));
    p = add(mul(p, s2), quo(1.0, 17.0));
    p = add(mul(p, s2), quo(1.0, 15.0));
    p = add(mul(p, s2), quo(1.0, 13.0));
    p = add(mul(p, s2), quo(1.0, 11.0));
    p = add(mul(p, s2), quo(1.0, 9.0));
    p = add(mul(p, s2), quo(1.0, 7.0));
    p = add(mul(p, s2), quo(1.0, 5.0));
    p = add(mul(p, s2), quo(1.0, 3.0));
    p = add(mul(p, s2), 1.0);
    return add(mul((double)(e - 53), 0.6931471805599453), mul(mul(2.0, s), p));
}

// cos(2 pi n 2^-53) for an integer n in [0, 2^53): the top three bits name the octant, the rest an angle of at most
// pi/4 (measured from the octant's nearer axis), whose cosine and sine are their series up to the 16th / 17th power.
Q6K_HD double cos_of_uniform(uint64_t n) {
    const int oct = (int)(n >> 50);
    uint64_t f = n & ((1ULL << 50) - 1);
    if (oct & 1) f = (1ULL << 50) - f;
    const double x = mul(mul((double)f, 8.8817841970012523e-16), 0.78539816339744831);      // f * 2^-50 * pi/4
    const double x2 = mul(x, x);
    const bool sine = oct == 1 || oct == 2 || oct == 5 || oct == 6;
    const bool minus = oct >= 2 && oct <= 5;
    double v;
    if (sine) {                                                     // x (1 - x2/3! + x4/5! - ... + x16/17!)
        double p = quo(1.0, 355687428096000.0);
        p = add(mul(p, x2), quo(-1.0, 1307674368000.0));
        p = add(mul(p, x2), quo(1.0, 6227020800.0));
        p = add(mul(p, x2), quo(-1.0, 39916800.0));
        p = add(mul(p, x2), quo(1.0, 362880.0));
        p = add(mul(p, x2), quo(-1.0, 5040.0));
        p = add(mul(p, x2), quo(1.0, 120.0));
        p = add(mul(p, x2), quo(-1.0, 6.0));
        p = add(mul(p, x2), 1.0);
        v = mul(x, p);
    } else {                                                        // 1 - x2/2! + x4/4! - ... + x16/16!
        double p = quo(1.0, 20922789888000.0);
        p = add(mul(p, x2), quo(-1.0, 87178291200.0));
        p = add(mul(p, x2), quo(1.0, 479001600.0));
        p = add(mul(p, x2), quo(-1.0, 3628800.0));
        p = add(mul(p, x2), quo(1.0, 40320.0));
        p = add(mul(p, x2), quo(-1.0, 720.0));
        p = add(mul(p, x2), quo(1.0, 24.0));
        p = add(mul(p, x2), quo(-1.0, 2.0));
        v = add(mul(p, x2), 1.0);
    }
    return minus ? -v : v;
}

// Element j of the N(0, 1) stream with the given key, as a float.
Q6K_HD float standard_normal(uint64_t key, uint64_t j) {
    const uint64_t a = mix(2 * j + key), b = mix(2 * j + 1 + key);
    const double r = root(mul(-2.0, log_of_uniform((a >> 11) + 1)));
    return (float)mul(r, cos_of_uniform(b >> 11));
}

// The element as it is stored before the cast to the tensor's dtype: z * std (+ mean), in float arithmetic.
Q6K_HD float element(uint64_t key, uint64_t j, float std, float mean) { return addf(mulf(standard_normal(key, j), std), mean); }

}  // namespace q6k_fill
