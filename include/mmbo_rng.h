/*
 * mmbo_rng.h -- counter-based generator for synthetic GEMM operands.
 *
 * Every matrix element is a pure function of (seed, matrix id, logical row, logical
 * column, logical row count): it does not depend on the leading dimension, on how the
 * matrix is sharded into column blocks, or on which processor evaluates it.  The same
 * header compiles as C, C++ and CUDA, and every floating-point operation in it is an
 * individually rounded IEEE-754 binary64 operation in a fixed order (explicit fma, no
 * library log/exp), so a host build and a device build return bit-identical values.
 *
 * Host translation units that include this header must be compiled with
 * -ffp-contract=off (the build recipes in this repository do so).
 *
 * The reference harness fills its operands with unseeded rand()/RAND_MAX
 * (src/gemm/benchmark.cc:44-52, src/gemm/test.cc:39-50); this generator replaces it
 * so that CPU and GPU runs see identical inputs.
 */
#ifndef MMBO_RNG_H_
#define MMBO_RNG_H_

#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define MMBO_HD __host__ __device__ __forceinline__
#else
#define MMBO_HD static inline
#endif

#if defined(__CUDA_ARCH__)
#define MMBO_MUL(a, b) __dmul_rn((a), (b))
#define MMBO_ADD(a, b) __dadd_rn((a), (b))
#define MMBO_DIV(a, b) __ddiv_rn((a), (b))
#define MMBO_FMA(a, b, c) __fma_rn((a), (b), (c))
#define MMBO_SQRT(a) __dsqrt_rn((a))
#else
#include <math.h>
#define MMBO_MUL(a, b) ((a) * (b))
#define MMBO_ADD(a, b) ((a) + (b))
#define MMBO_DIV(a, b) ((a) / (b))
#define MMBO_FMA(a, b, c) fma((a), (b), (c))
#define MMBO_SQRT(a) sqrt((a))
#endif

/* Distributions. */
#define MMBO_DIST_UNIFORM_PM1 0 /* uniform on [-1, 1), scaled by `scale`            */
#define MMBO_DIST_NORMAL 1      /* normal(0, 1) scaled by `scale` (= the std. dev.) */
#define MMBO_DIST_ZERO 2        /* all zeros                                        */

/* Matrix ids used by the harness and the tests. */
#define MMBO_MAT_A 0
#define MMBO_MAT_B 1
#define MMBO_MAT_C 2

/* splitmix64 finaliser. */
MMBO_HD uint64_t mmbo_mix64(uint64_t z) {
  z ^= z >> 30;
  z *= 0xbf58476d1ce4e5b9ull;
  z ^= z >> 27;
  z *= 0x94d049bb133111ebull;
  z ^= z >> 31;
  return z;
}

/* 64 random bits for element `idx` (= row + col * rows) of matrix `mat`. */
MMBO_HD uint64_t mmbo_bits(uint64_t seed, uint32_t mat, uint64_t idx) {
  uint64_t key = mmbo_mix64(seed + 0x9e3779b97f4a7c15ull * (uint64_t)(mat + 1u));
  return mmbo_mix64(key ^ (idx * 0xd1342543de82ef95ull + 0x2545f4914f6cdd1dull));
}

MMBO_HD double mmbo_from_bits(uint64_t u) {
  double d;
#if defined(__CUDA_ARCH__)
  d = __longlong_as_double((long long)u);
#else
  memcpy(&d, &u, sizeof d);
#endif
  return d;
}

MMBO_HD uint64_t mmbo_to_bits(double d) {
#if defined(__CUDA_ARCH__)
  return (uint64_t)__double_as_longlong(d);
#else
  uint64_t u;
  memcpy(&u, &d, sizeof u);
  return u;
#endif
}

/* Natural logarithm of a positive normal double from individually rounded operations:
 * x = m * 2^e with m in [sqrt(1/2), sqrt(2)), log m = 2 atanh(s), s = (m-1)/(m+1),
 * odd series in s up to s^23 (truncation below 1e-18 since |s| < 0.1716). */
MMBO_HD double mmbo_log(double x) {
  uint64_t u = mmbo_to_bits(x);
  int e = (int)((u >> 52) & 0x7ff) - 1023;
  double m = mmbo_from_bits((u & 0x000fffffffffffffull) | 0x3ff0000000000000ull);
  if (m > 1.4142135623730951) {
    m = MMBO_MUL(m, 0.5);
    e += 1;
  }
  double s = MMBO_DIV(MMBO_ADD(m, -1.0), MMBO_ADD(m, 1.0));
  double s2 = MMBO_MUL(s, s);
  double p = 1.0 / 23.0;
  p = MMBO_FMA(p, s2, 1.0 / 21.0);
  p = MMBO_FMA(p, s2, 1.0 / 19.0);
  p = MMBO_FMA(p, s2, 1.0 / 17.0);
  p = MMBO_FMA(p, s2, 1.0 / 15.0);
  p = MMBO_FMA(p, s2, 1.0 / 13.0);
  p = MMBO_FMA(p, s2, 1.0 / 11.0);
  p = MMBO_FMA(p, s2, 1.0 / 9.0);
  p = MMBO_FMA(p, s2, 1.0 / 7.0);
  p = MMBO_FMA(p, s2, 1.0 / 5.0);
  p = MMBO_FMA(p, s2, 1.0 / 3.0);
  p = MMBO_FMA(p, s2, 1.0);
  double lm = MMBO_MUL(MMBO_MUL(2.0, s), p);
  return MMBO_FMA((double)e, 0.6931471805599453, lm);
}

/* Inverse of the standard normal CDF (P. J. Acklam's rational approximation,
 * relative error below 1.2e-9), p in (0, 1). */
MMBO_HD double mmbo_norminv(double p) {
  const double a1 = -3.969683028665376e+01, a2 = 2.209460984245205e+02,
               a3 = -2.759285104469687e+02, a4 = 1.383577518672690e+02,
               a5 = -3.066479806614716e+01, a6 = 2.506628277459239e+00;
  const double b1 = -5.447609879822406e+01, b2 = 1.615858368580409e+02,
               b3 = -1.556989798598866e+02, b4 = 6.680131188771972e+01,
               b5 = -1.328068155288572e+01;
  const double c1 = -7.784894002430293e-03, c2 = -3.223964580411365e-01,
               c3 = -2.400758277161838e+00, c4 = -2.549732539343734e+00,
               c5 = 4.374664141464968e+00, c6 = 2.938163982698783e+00;
  const double d1 = 7.784695709041462e-03, d2 = 3.224671290700398e-01,
               d3 = 2.445134137142996e+00, d4 = 3.754408661907416e+00;
  const double plow = 0.02425;
  if (p < plow || p > 1.0 - plow) {
    int upper = p > 0.5;
    double pp = upper ? MMBO_ADD(1.0, -p) : p;
    double q = MMBO_SQRT(MMBO_MUL(-2.0, mmbo_log(pp)));
    double num = c1;
    num = MMBO_FMA(num, q, c2);
    num = MMBO_FMA(num, q, c3);
    num = MMBO_FMA(num, q, c4);
    num = MMBO_FMA(num, q, c5);
    num = MMBO_FMA(num, q, c6);
    double den = d1;
    den = MMBO_FMA(den, q, d2);
    den = MMBO_FMA(den, q, d3);
    den = MMBO_FMA(den, q, d4);
    den = MMBO_FMA(den, q, 1.0);
    double x = MMBO_DIV(num, den);
    return upper ? -x : x;
  } else {
    double q = MMBO_ADD(p, -0.5);
    double r = MMBO_MUL(q, q);
    double num = a1;
    num = MMBO_FMA(num, r, a2);
    num = MMBO_FMA(num, r, a3);
    num = MMBO_FMA(num, r, a4);
    num = MMBO_FMA(num, r, a5);
    num = MMBO_FMA(num, r, a6);
    double den = b1;
    den = MMBO_FMA(den, r, b2);
    den = MMBO_FMA(den, r, b3);
    den = MMBO_FMA(den, r, b4);
    den = MMBO_FMA(den, r, b5);
    den = MMBO_FMA(den, r, 1.0);
    return MMBO_DIV(MMBO_MUL(num, q), den);
  }
}

/* Value of element (row, col) of a `rows`-row matrix, as a float (exactly rounded
 * from the binary64 intermediate). */
MMBO_HD float mmbo_rng_value(uint64_t seed, uint32_t mat, uint64_t row, uint64_t col,
                             uint64_t rows, int dist, float scale) {
  if (dist == MMBO_DIST_ZERO) return 0.0f;
  uint64_t h = mmbo_bits(seed, mat, row + col * rows);
  if (dist == MMBO_DIST_UNIFORM_PM1) {
    /* 24 random bits -> multiple of 2^-23 in [-1, 1): exact in binary32. */
    float u = (float)(uint32_t)(h >> 40) * 1.1920928955078125e-07f - 1.0f;
    return u * scale;
  }
  /* 53 random bits + 1/2 -> p in (0, 1), never 0 or 1. */
  double p = MMBO_MUL(MMBO_ADD((double)(h >> 11), 0.5), 1.1102230246251565e-16);
  double z = MMBO_MUL(mmbo_norminv(p), (double)scale);
  return (float)z;
}

/* IEEE binary16 <-> binary32 conversions (round to nearest even), usable where the
 * compiler has no native half type. */
MMBO_HD uint16_t mmbo_f32_to_f16_bits(float f) {
  uint32_t x;
#if defined(__CUDA_ARCH__)
  x = __float_as_uint(f);
#else
  memcpy(&x, &f, sizeof x);
#endif
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t ax = x & 0x7fffffffu;
  if (ax >= 0x7f800000u) { /* inf / nan */
    return (uint16_t)(sign | 0x7c00u | ((ax > 0x7f800000u) ? 0x0200u : 0u));
  }
  if (ax >= 0x477ff000u) { /* rounds to >= 65520 -> inf */
    return (uint16_t)(sign | 0x7c00u);
  }
  if (ax < 0x33000001u) { /* <= 2^-25 -> zero */
    return (uint16_t)sign;
  }
  uint32_t e = ax >> 23;
  uint32_t mant = (ax & 0x007fffffu) | 0x00800000u;
  uint32_t shift, half_exp;
  if (e >= 113) { /* normal half */
    shift = 13;
    half_exp = e - 112;
  } else { /* subnormal half */
    shift = 126 - e;
    half_exp = 0;
  }
  uint32_t q = mant >> shift;
  uint32_t rem = mant & ((1u << shift) - 1u);
  uint32_t halfway = 1u << (shift - 1);
  if (rem > halfway || (rem == halfway && (q & 1u))) q += 1;
  uint32_t out;
  if (half_exp) out = ((half_exp - 1) << 10) + q; /* q carries the implicit bit */
  else out = q;
  return (uint16_t)(sign | out);
}

MMBO_HD float mmbo_f16_bits_to_f32(uint16_t h) {
  uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  uint32_t e = (h >> 10) & 0x1fu;
  uint32_t m = h & 0x3ffu;
  uint32_t x;
  if (e == 0) {
    if (m == 0) {
      x = sign;
    } else {
      int s = 0;
      while (!(m & 0x400u)) {
        m <<= 1;
        s++;
      }
      x = sign | ((uint32_t)(113 - s) << 23) | ((m & 0x3ffu) << 13);
    }
  } else if (e == 31) {
    x = sign | 0x7f800000u | (m << 13);
  } else {
    x = sign | ((e + 112) << 23) | (m << 13);
  }
  float f;
#if defined(__CUDA_ARCH__)
  f = __uint_as_float(x);
#else
  memcpy(&f, &x, sizeof f);
#endif
  return f;
}

#endif /* MMBO_RNG_H_ */
