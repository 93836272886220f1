// Seeded random weights: one counter-based generator for the host and the device.
//
// Element i of the tensor called `name` under `seed` is a function of (seed, name, i) alone, so its value
// depends neither on the order in which tensors are made, nor on which other tensors exist, nor on whether the
// host wrote it into a safetensors file or the device filled it in place: random_value() below is compiled for
// both and gives the same bits on both, because it uses only IEEE-754 additions, multiplications, divisions and
// square roots in double precision, none of them contracted into a fused multiply-add (the device code calls
// the _rn intrinsics, the host library is compiled with -ffp-contract=off).  Logarithm, sine and cosine are
// short series here for that reason, not library calls.
//
// The reference has no such mode in its engine; it makes tiny checkpoints offline with another framework
// (tools/gen_tiny_ckpt.py:53-61).
#pragma once

#include <stdint.h>

#if defined(__CUDACC__)
#define QE_HD __host__ __device__ __forceinline__
#else
#define QE_HD inline
#endif

namespace qe {
namespace rnd {

#if defined(__CUDA_ARCH__)
QE_HD double mul(double a, double b) { return __dmul_rn(a, b); }
QE_HD double add(double a, double b) { return __dadd_rn(a, b); }
QE_HD double div(double a, double b) { return __ddiv_rn(a, b); }
QE_HD double root(double a) { return __dsqrt_rn(a); }
#else
QE_HD double mul(double a, double b) { return a * b; }
QE_HD double add(double a, double b) { return a + b; }
QE_HD double div(double a, double b) { return a / b; }
QE_HD double root(double a) { return __builtin_sqrt(a); }
#endif

// The finaliser of splitmix64 (a bijection of 64-bit words with good avalanche).
QE_HD uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}

// The key of one tensor: the seed and the FNV-1a hash of its name, mixed.
inline uint64_t tensor_key(uint64_t seed, const char* name) {
    uint64_t h = 0xCBF29CE484222325ULL;
    for (const unsigned char* p = (const unsigned char*)name; *p; p++) h = (h ^ *p) * 0x100000001B3ULL;
    return mix64(mix64(seed + 0x9E3779B97F4A7C15ULL) ^ h);
}

// Word k (0 or 1) of element i.
QE_HD uint64_t word(uint64_t key, uint64_t i, uint64_t k) { return mix64(key + (2 * i + k + 1) * 0x9E3779B97F4A7C15ULL); }

// ln(n * 2^-53) for an integer n in [1, 2^53].
QE_HD double log_unit(uint64_t n) {
#if defined(__CUDA_ARCH__)
    int b = 63 - __clzll((long long)n);                     // highest set bit
#else
    int b = 63 - __builtin_clzll(n);
#endif
    double m = mul((double)n, 1.0 / (double)(1ULL << b));   // in [1, 2), exact
    if (m > 1.4142135623730951) { m = mul(m, 0.5); b++; }
    const double s = div(add(m, -1.0), add(m, 1.0));        // |s| <= 0.1716; ln m = 2 atanh s
    const double s2 = mul(s, s);
    double acc = 1.0 / 25.0;
    acc = add(mul(acc, s2), 1.0 / 23.0);
    acc = add(mul(acc, s2), 1.0 / 21.0);
    acc = add(mul(acc, s2), 1.0 / 19.0);
    acc = add(mul(acc, s2), 1.0 / 17.0);
    acc = add(mul(acc, s2), 1.0 / 15.0);
    acc = add(mul(acc, s2), 1.0 / 13.0);
    acc = add(mul(acc, s2), 1.0 / 11.0);
    acc = add(mul(acc, s2), 1.0 / 9.0);
    acc = add(mul(acc, s2), 1.0 / 7.0);
    acc = add(mul(acc, s2), 1.0 / 5.0);
    acc = add(mul(acc, s2), 1.0 / 3.0);
    acc = add(mul(acc, s2), 1.0);
    const double ln_m = mul(2.0, mul(s, acc));
    return add(ln_m, mul((double)(b - 53), 0.6931471805599453));
}

// cos and sin of t in [0, pi/4] by their Taylor series.
QE_HD double cos_small(double t) {
    const double x = mul(t, t);
    double acc = 1.0 / 6402373705728000.0;                 // 1/18!
    acc = add(mul(acc, -x), 1.0 / 20922789888000.0);        // 1/16!
    acc = add(mul(acc, -x), 1.0 / 87178291200.0);           // 1/14!
    acc = add(mul(acc, -x), 1.0 / 479001600.0);             // 1/12!
    acc = add(mul(acc, -x), 1.0 / 3628800.0);               // 1/10!
    acc = add(mul(acc, -x), 1.0 / 40320.0);                 // 1/8!
    acc = add(mul(acc, -x), 1.0 / 720.0);
    acc = add(mul(acc, -x), 1.0 / 24.0);
    acc = add(mul(acc, -x), 0.5);
    return add(mul(acc, -x), 1.0);
}
QE_HD double sin_small(double t) {
    const double x = mul(t, t);
    double acc = 1.0 / 121645100408832000.0;               // 1/19!
    acc = add(mul(acc, -x), 1.0 / 355687428096000.0);       // 1/17!
    acc = add(mul(acc, -x), 1.0 / 1307674368000.0);         // 1/15!
    acc = add(mul(acc, -x), 1.0 / 6227020800.0);            // 1/13!
    acc = add(mul(acc, -x), 1.0 / 39916800.0);              // 1/11!
    acc = add(mul(acc, -x), 1.0 / 362880.0);                // 1/9!
    acc = add(mul(acc, -x), 1.0 / 5040.0);
    acc = add(mul(acc, -x), 1.0 / 120.0);
    acc = add(mul(acc, -x), 1.0 / 6.0);
    acc = add(mul(acc, -x), 1.0);
    return mul(t, acc);
}

// cos(2 pi n 2^-53) for n in [0, 2^53): the top three bits pick the octant, the rest the angle inside it.
QE_HD double cos_turn(uint64_t n) {
    const int octant = (int)(n >> 50);
    const uint64_t frac = n & ((1ULL << 50) - 1);
    const double f = mul((double)frac, 1.0 / (double)(1ULL << 50));
    const double quarter_pi = 0.7853981633974483;
    const double t = mul((octant & 1) ? add(1.0, -f) : f, quarter_pi);
    switch (octant) {
        case 0: return cos_small(t);
        case 1: return sin_small(t);
        case 2: return -sin_small(t);
        case 3: return -cos_small(t);
        case 4: return -cos_small(t);
        case 5: return -sin_small(t);
        case 6: return sin_small(t);
        default: return cos_small(t);
    }
}

// A standard normal value (Box-Muller, the cosine branch).
QE_HD double standard_normal(uint64_t key, uint64_t i) {
    const uint64_t n1 = (word(key, i, 0) >> 11) + 1;        // (0, 1] in units of 2^-53
    const uint64_t n2 = word(key, i, 1) >> 11;              // [0, 1)
    const double r = root(mul(-2.0, log_unit(n1)));
    return mul(r, cos_turn(n2));
}
QE_HD double uniform_unit(uint64_t key, uint64_t i) { return mul((double)(word(key, i, 0) >> 11), 1.0 / 9007199254740992.0); }

// kind 0: N(0, a); kind 1: U(a, b); kind 2: the constant a.
QE_HD float random_value(uint64_t key, uint64_t i, int kind, double a, double b) {
    if (kind == 0) return (float)mul(standard_normal(key, i), a);
    if (kind == 1) return (float)add(a, mul(add(b, -a), uniform_unit(key, i)));
    return (float)a;
}

}  // namespace rnd
}  // namespace qe
