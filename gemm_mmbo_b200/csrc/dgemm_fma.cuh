// DGEMM on the CUDA cores (DFMA): C = alpha * op(A) * op(B) + beta * C in binary64 --
// the reference's own data type (src/gemm/gemm.h:4,47 take double; its kernels are
// v_fma_f64 loops, e.g. src/gemm/assembly/naive_gemm_kernel_64_64_4_4.s).  Macro-tile
// 64 x 64 x 16 with a 4 x 4 micro-tile per thread and 256 threads, i.e. the shape of the
// reference's MT064x064 kernels (src/gemm/constants.h:36), double-buffered shared
// memory, register prefetch of the next slab, guarded loads with zero-filled tails,
// all four transpose modes and any leading dimensions.  The write rule is the
// reference's (src/gemm/ref/Kernels.cpp:87).  On this GPU the DFMA pipe issues 64
// lanes per SM per clock, so a plain register-blocked kernel is bound by that pipe.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "raster.h"

namespace mmbo {

struct DgemmParams {
  uint32_t m, n, k;
  uint32_t lda, ldb, ldc;
  double alpha, beta;
  uint32_t wgm;
  uint32_t diag;  // diagnostic runs only (bit 0: no C traffic; results wrong by design), never set in production
  uint32_t tma_a, tma_b;  // warp-specialised kernel: the operand is addressed through its tensor map
  uint32_t tma_c;         // ... and the old C can be staged through shared memory (64-row tiles)
  // strided batch (src/gemm/ref/Kernels.cpp:254 takes the problem index from the grid): number of
  // problems and the elements between consecutive problems' A, B, C
  uint32_t batch;
  unsigned long long batch_a, batch_b, batch_c;
};

constexpr int kDgBM = 64, kDgBN = 64, kDgBK = 16, kDgThreads = 256;

// Loads a 64 x 16 slab of an operand (4 elements per thread).  CONTIG_ROW: the tile-row
// index (m or n) is the contiguous one in memory.
template <bool CONTIG_ROW>
__device__ __forceinline__ void dg_load(double (&reg)[4], const double* __restrict__ base, uint32_t ld,
                                        uint32_t row0, uint32_t l0, uint32_t row_end, uint32_t l_end, int tid) {
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int idx = tid + e * kDgThreads;
    const uint32_t row = CONTIG_ROW ? idx % kDgBM : idx / kDgBK;
    const uint32_t l = CONTIG_ROW ? idx / kDgBM : idx % kDgBK;
    double x = 0.0;
    if (row0 + row < row_end && l0 + l < l_end) {
      const size_t off = CONTIG_ROW ? (size_t)(row0 + row) + (size_t)(l0 + l) * ld
                                    : (size_t)(l0 + l) + (size_t)(row0 + row) * ld;
      x = __ldg(base + off);
    }
    reg[e] = x;
  }
}

// Shared tile layout [16][64 + 2] doubles (row index contiguous).
template <bool CONTIG_ROW>
__device__ __forceinline__ void dg_store(const double (&reg)[4], double* __restrict__ tile, int tid) {
  constexpr int kPitch = kDgBM + 2;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int idx = tid + e * kDgThreads;
    const int row = CONTIG_ROW ? idx % kDgBM : idx / kDgBK;
    const int l = CONTIG_ROW ? idx / kDgBM : idx % kDgBK;
    tile[l * kPitch + row] = reg[e];
  }
}

template <bool TRANS_A, bool TRANS_B>
__global__ void __launch_bounds__(kDgThreads, 2)
dgemm_fma_kernel(const double* __restrict__ A, const double* __restrict__ B, double* __restrict__ C,
                 const DgemmParams p) {
  constexpr int kPitch = kDgBM + 2;
  __shared__ __align__(16) double sA[2][kDgBK * kPitch];
  __shared__ __align__(16) double sB[2][kDgBK * kPitch];
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;  // lanes run along m
  A += (size_t)blockIdx.z * p.batch_a;  // problem blockIdx.z of a strided batch
  B += (size_t)blockIdx.z * p.batch_b;
  C += (size_t)blockIdx.z * p.batch_c;

  uint32_t tile_m, tile_n;
  mmbo_wgm_remap(blockIdx.x, blockIdx.y, gridDim.x, gridDim.y, p.wgm, &tile_m, &tile_n);
  const uint32_t m0 = tile_m * kDgBM, n0 = tile_n * kDgBN;

  double acc[4][4];
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[j][i] = 0.0;

  double ra[4], rb[4];
  const uint32_t num_kb = (p.k + kDgBK - 1) / kDgBK;
  dg_load<!TRANS_A>(ra, A, p.lda, m0, 0, p.m, p.k, tid);
  dg_load<TRANS_B>(rb, B, p.ldb, n0, 0, p.n, p.k, tid);
  dg_store<!TRANS_A>(ra, sA[0], tid);
  dg_store<TRANS_B>(rb, sB[0], tid);
  __syncthreads();

  for (uint32_t kb = 0; kb < num_kb; ++kb) {
    const int cur = kb & 1;
    if (kb + 1 < num_kb) {
      dg_load<!TRANS_A>(ra, A, p.lda, m0, (kb + 1) * kDgBK, p.m, p.k, tid);
      dg_load<TRANS_B>(rb, B, p.ldb, n0, (kb + 1) * kDgBK, p.n, p.k, tid);
    }
    const double* __restrict__ a_s = sA[cur];
    const double* __restrict__ b_s = sB[cur];
#pragma unroll
    for (int l = 0; l < kDgBK; ++l) {
      // micro-tile rows {2tx, 2tx+1, 32+2tx, 33+2tx}: two 16-byte pieces 32 elements apart
      const double2 a0 = *reinterpret_cast<const double2*>(a_s + l * kPitch + tx * 2);
      const double2 a1 = *reinterpret_cast<const double2*>(a_s + l * kPitch + 32 + tx * 2);
      const double2 b0 = *reinterpret_cast<const double2*>(b_s + l * kPitch + ty * 2);
      const double2 b1 = *reinterpret_cast<const double2*>(b_s + l * kPitch + 32 + ty * 2);
      const double fa[4] = {a0.x, a0.y, a1.x, a1.y};
      const double fb[4] = {b0.x, b0.y, b1.x, b1.y};
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = fma(fa[i], fb[j], acc[j][i]);
    }
    if (kb + 1 < num_kb) {
      dg_store<!TRANS_A>(ra, sA[cur ^ 1], tid);
      dg_store<TRANS_B>(rb, sB[cur ^ 1], tid);
    }
    __syncthreads();
  }

  const double alpha = p.alpha, beta = p.beta;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t nj = n0 + (j >> 1) * 32 + ty * 2 + (j & 1);
    if (nj >= p.n) continue;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t mi = m0 + (i >> 1) * 32 + tx * 2 + (i & 1);
      if (mi >= p.m) continue;
      double* cp = C + (size_t)mi + (size_t)nj * p.ldc;
      double r = alpha * acc[j][i];
      if (beta != 0.0) r = fma(beta, *cp, r);
      *cp = r;
    }
  }
}

}  // namespace mmbo
