/*
 * ref_gemm.c -- CPU oracle for the GEMM hot path.  TEST INFRASTRUCTURE ONLY: nothing
 * in the shipped library calls, links or imports this file.  It is used by tests/, by
 * the smoke check and as the timed CPU baseline of the benchmark.
 *
 * Parity status: the reference (CSWater/GEMM_MMBO) has no CPU GEMM and no golden GEMM
 * vectors; its only numeric check compares a GPU kernel with rocBLAS rocblas_dgemm
 * (third party, linked from /opt/rocm with no version pinned: src/gemm/Makefile:4,7,
 * call sites src/gemm/test.cc:95-101) on unseeded inputs at |diff| <= 1e-5
 * (src/gemm/test.cc:12,109-115).  GEMM numeric parity is therefore UNPINNED; what is
 * pinned by a reference golden vector is the work-group remap (see wgm_map.c).
 *
 * What this file restates:
 *   - the per-element arithmetic  acc += A*B ;  C = beta != 0 ? alpha*acc + beta*C
 *     : alpha*acc   (src/gemm/ref/Kernels.cpp:84-87, MAC / TYPE_MAC_WRITE); with
 *     beta == 0 the old C is never read, so NaN/Inf in it do not propagate;
 *   - column-major addressing C[i + j*ldc], A[i + l*lda], B[j + l*ldb] for the
 *     reference's NT case (src/gemm/ref/Kernels.cpp:76-78, strides from
 *     src/gemm/gemm.h:81-90, operand shapes src/gemm/benchmark.cc:26,40-42), extended
 *     to NN/TN/TT by the BLAS op() convention:
 *       op(A)(i,l) = transA ? A[l + i*lda] : A[i + l*lda]
 *       op(B)(l,j) = transB ? B[j + l*ldb] : B[l + j*ldb]
 *   - accumulation in binary64 whatever the storage type, in increasing l.
 *
 * Two implementations are provided and tested against each other for bit equality:
 * oracle_gemm_naive_* (the literal triple loop) and oracle_gemm_* (packed, register
 * blocked, OpenMP over column panels; every C element still sums its k products in
 * increasing l, so the result is bit-identical to the naive loop).
 */
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#include "mmbo_rng.h"

#define DT_F32 0
#define DT_F16 1
#define DT_F64 2

static inline double load_elem(const void *p, size_t idx, int dt) {
  if (dt == DT_F32) return (double)((const float *)p)[idx];
  if (dt == DT_F64) return ((const double *)p)[idx];
  return (double)mmbo_f16_bits_to_f32(((const uint16_t *)p)[idx]);
}

/* ---- literal triple loop ------------------------------------------------------- */
static void gemm_naive(int dt, int transA, int transB, size_t m, size_t n, size_t k,
                       double alpha, const void *A, size_t lda, const void *B, size_t ldb,
                       double beta, const void *Cin, size_t ldc, double *Cout,
                       size_t ldo) {
  for (size_t j = 0; j < n; ++j) {
    for (size_t i = 0; i < m; ++i) {
      double acc = 0.0;
      for (size_t l = 0; l < k; ++l) {
        double a = load_elem(A, transA ? l + i * lda : i + l * lda, dt);
        double b = load_elem(B, transB ? j + l * ldb : l + j * ldb, dt);
        acc += a * b;
      }
      double r;
      if (beta != 0.0) r = alpha * acc + beta * load_elem(Cin, i + j * ldc, dt);
      else r = alpha * acc;
      Cout[i + j * ldo] = r;
    }
  }
}

/* ---- packed / blocked / threaded ------------------------------------------------ */
#define MR 4
#define NR 8

#if defined(ORACLE_CLONES) && defined(__x86_64__)
__attribute__((target_clones("avx2", "default")))
#endif
static void gemm_blocked(int dt, int transA, int transB, size_t m, size_t n, size_t k,
                         double alpha, const void *A, size_t lda, const void *B,
                         size_t ldb, double beta, const void *Cin, size_t ldc,
                         double *Cout, size_t ldo) {
  if (m == 0 || n == 0) return;
  const size_t mp = (m + MR - 1) / MR * MR;
  const size_t np = (n + NR - 1) / NR * NR;
  /* Ap: [mp/MR][k][MR]; Bp: [np/NR][k][NR]; zero padded. */
  double *Ap = (double *)calloc(mp * (k ? k : 1), sizeof(double));
  double *Bp = (double *)calloc(np * (k ? k : 1), sizeof(double));
  if (!Ap || !Bp) abort();
#pragma omp parallel for schedule(static)
  for (ptrdiff_t ib = 0; ib < (ptrdiff_t)(mp / MR); ++ib)
    for (size_t l = 0; l < k; ++l)
      for (size_t r = 0; r < MR; ++r) {
        size_t i = (size_t)ib * MR + r;
        if (i < m)
          Ap[((size_t)ib * k + l) * MR + r] =
              load_elem(A, transA ? l + i * lda : i + l * lda, dt);
      }
#pragma omp parallel for schedule(static)
  for (ptrdiff_t jb = 0; jb < (ptrdiff_t)(np / NR); ++jb)
    for (size_t l = 0; l < k; ++l)
      for (size_t c = 0; c < NR; ++c) {
        size_t j = (size_t)jb * NR + c;
        if (j < n)
          Bp[((size_t)jb * k + l) * NR + c] =
              load_elem(B, transB ? j + l * ldb : l + j * ldb, dt);
      }
#pragma omp parallel for schedule(dynamic, 4)
  for (ptrdiff_t jb = 0; jb < (ptrdiff_t)(np / NR); ++jb) {
    const double *bp = Bp + (size_t)jb * k * NR;
    for (size_t ib = 0; ib < mp / MR; ++ib) {
      const double *ap = Ap + ib * k * MR;
      double acc[MR][NR];
      for (int r = 0; r < MR; ++r)
        for (int c = 0; c < NR; ++c) acc[r][c] = 0.0;
      for (size_t l = 0; l < k; ++l) {
        const double *a = ap + l * MR;
        const double *b = bp + l * NR;
        for (int r = 0; r < MR; ++r)
          for (int c = 0; c < NR; ++c) acc[r][c] += a[r] * b[c];
      }
      for (int c = 0; c < NR; ++c) {
        size_t j = (size_t)jb * NR + c;
        if (j >= n) break;
        for (int r = 0; r < MR; ++r) {
          size_t i = ib * MR + r;
          if (i >= m) break;
          double v;
          if (beta != 0.0) v = alpha * acc[r][c] + beta * load_elem(Cin, i + j * ldc, dt);
          else v = alpha * acc[r][c];
          Cout[i + j * ldo] = v;
        }
      }
    }
  }
  free(Ap);
  free(Bp);
}

/* ---- exported entry points -------------------------------------------------------
 * A, B, Cin are host arrays of the storage type; Cout is an m x n binary64 array with
 * leading dimension ldo (the unrounded result).  alpha and beta are the values the
 * GPU library receives (binary32), widened. */
void oracle_gemm_f32(int transA, int transB, size_t m, size_t n, size_t k, float alpha,
                     const float *A, size_t lda, const float *B, size_t ldb, float beta,
                     const float *Cin, size_t ldc, double *Cout, size_t ldo) {
  gemm_blocked(DT_F32, transA, transB, m, n, k, (double)alpha, A, lda, B, ldb,
               (double)beta, Cin, ldc, Cout, ldo);
}

void oracle_gemm_f16(int transA, int transB, size_t m, size_t n, size_t k, float alpha,
                     const uint16_t *A, size_t lda, const uint16_t *B, size_t ldb,
                     float beta, const uint16_t *Cin, size_t ldc, double *Cout,
                     size_t ldo) {
  gemm_blocked(DT_F16, transA, transB, m, n, k, (double)alpha, A, lda, B, ldb,
               (double)beta, Cin, ldc, Cout, ldo);
}

void oracle_gemm_naive_f32(int transA, int transB, size_t m, size_t n, size_t k,
                           float alpha, const float *A, size_t lda, const float *B,
                           size_t ldb, float beta, const float *Cin, size_t ldc,
                           double *Cout, size_t ldo) {
  gemm_naive(DT_F32, transA, transB, m, n, k, (double)alpha, A, lda, B, ldb,
             (double)beta, Cin, ldc, Cout, ldo);
}

void oracle_gemm_naive_f16(int transA, int transB, size_t m, size_t n, size_t k,
                           float alpha, const uint16_t *A, size_t lda, const uint16_t *B,
                           size_t ldb, float beta, const uint16_t *Cin, size_t ldc,
                           double *Cout, size_t ldo) {
  gemm_naive(DT_F16, transA, transB, m, n, k, (double)alpha, A, lda, B, ldb,
             (double)beta, Cin, ldc, Cout, ldo);
}

/* binary64 storage (the reference's own dtype: src/gemm/gemm.h:4,47 take double).  A
 * binary64 accumulator would be no more accurate than the kernel under test, so this
 * one accumulates in long double (64-bit significand on x86-64) in increasing l. */
void oracle_gemm_f64(int transA, int transB, size_t m, size_t n, size_t k, double alpha,
                     const double *A, size_t lda, const double *B, size_t ldb, double beta,
                     const double *Cin, size_t ldc, double *Cout, size_t ldo) {
#pragma omp parallel for schedule(dynamic, 1)
  for (ptrdiff_t j = 0; j < (ptrdiff_t)n; ++j)
    for (size_t i = 0; i < m; ++i) {
      long double acc = 0.0L;
      for (size_t l = 0; l < k; ++l) {
        long double a = transA ? A[l + i * lda] : A[i + l * lda];
        long double b = transB ? B[(size_t)j + l * ldb] : B[l + (size_t)j * ldb];
        acc += a * b;
      }
      long double r = (long double)alpha * acc;
      if (beta != 0.0) r += (long double)beta * (long double)Cin[i + (size_t)j * ldc];
      Cout[i + (size_t)j * ldo] = (double)r;
    }
}

void oracle_fill_f64(double *dst, size_t rows, size_t cols, size_t ld, uint64_t seed,
                     uint32_t mat, int dist, float scale, size_t row0, size_t col0,
                     size_t total_rows) {
#pragma omp parallel for schedule(static)
  for (ptrdiff_t j = 0; j < (ptrdiff_t)cols; ++j)
    for (size_t i = 0; i < rows; ++i)
      dst[i + (size_t)j * ld] =
          (double)mmbo_rng_value(seed, mat, row0 + i, col0 + (size_t)j, total_rows, dist, scale);
}

/* Selected elements only: out[t] = element (rows[t], cols[t]) of the result.  Used to
 * check sizes whose full product is out of reach of host cores. */
void oracle_gemm_sampled(int dt, int transA, int transB, size_t k, float alpha,
                         const void *A, size_t lda, const void *B, size_t ldb, float beta,
                         const void *Cin, size_t ldc, size_t nsamples, const size_t *rows,
                         const size_t *cols, double *out) {
#pragma omp parallel for schedule(static)
  for (ptrdiff_t t = 0; t < (ptrdiff_t)nsamples; ++t) {
    size_t i = rows[t], j = cols[t];
    double acc = 0.0;
    for (size_t l = 0; l < k; ++l) {
      double a = load_elem(A, transA ? l + i * lda : i + l * lda, dt);
      double b = load_elem(B, transB ? j + l * ldb : l + j * ldb, dt);
      acc += a * b;
    }
    double a64 = (double)alpha, b64 = (double)beta;
    out[t] = (b64 != 0.0) ? a64 * acc + b64 * load_elem(Cin, i + j * ldc, dt) : a64 * acc;
  }
}

/* Relative Frobenius error || got - ref ||_F / || ref ||_F over an m x n window.
 * `got` has the storage type dt (0 = f32, 1 = f16 bits); NaN in `got` yields NaN. */
double oracle_rel_frobenius(int dt, size_t m, size_t n, const void *got, size_t ldg,
                            const double *ref, size_t ldr) {
  double num = 0.0, den = 0.0;
#pragma omp parallel for reduction(+ : num, den) schedule(static)
  for (ptrdiff_t j = 0; j < (ptrdiff_t)n; ++j) {
    double pn = 0.0, pd = 0.0;
    for (size_t i = 0; i < m; ++i) {
      double g = load_elem(got, i + (size_t)j * ldg, dt);
      double r = ref[i + (size_t)j * ldr];
      double d = g - r;
      pn += d * d;
      pd += r * r;
    }
    num += pn;
    den += pd;
  }
  if (den == 0.0) return num == 0.0 ? 0.0 : INFINITY;
  return sqrt(num / den);
}

/* Seeded operand generation (same generator the GPU library's fill kernels use).
 * Fills the rows x cols window of a column-major array with leading dimension ld;
 * padding rows (row >= rows) are left untouched. */
void oracle_fill_f32(float *dst, size_t rows, size_t cols, size_t ld, uint64_t seed,
                     uint32_t mat, int dist, float scale, size_t row0, size_t col0,
                     size_t total_rows) {
#pragma omp parallel for schedule(static)
  for (ptrdiff_t j = 0; j < (ptrdiff_t)cols; ++j)
    for (size_t i = 0; i < rows; ++i)
      dst[i + (size_t)j * ld] =
          mmbo_rng_value(seed, mat, row0 + i, col0 + (size_t)j, total_rows, dist, scale);
}

void oracle_fill_f16(uint16_t *dst, size_t rows, size_t cols, size_t ld, uint64_t seed,
                     uint32_t mat, int dist, float scale, size_t row0, size_t col0,
                     size_t total_rows) {
#pragma omp parallel for schedule(static)
  for (ptrdiff_t j = 0; j < (ptrdiff_t)cols; ++j)
    for (size_t i = 0; i < rows; ++i)
      dst[i + (size_t)j * ld] = mmbo_f32_to_f16_bits(
          mmbo_rng_value(seed, mat, row0 + i, col0 + (size_t)j, total_rows, dist, scale));
}

/* Thread count for the parallel loops (launchers such as torchrun export
 * OMP_NUM_THREADS=1; the CPU baseline wants every host core).  n <= 0: all cores. */
void oracle_set_num_threads(int n) {
#ifdef _OPENMP
  if (n <= 0) n = omp_get_num_procs();
  omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
