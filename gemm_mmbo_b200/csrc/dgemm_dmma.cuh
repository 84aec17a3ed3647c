// DGEMM on the fp64 tensor path: C = alpha * op(A) * op(B) + beta * C in binary64 with
// mma.sync.m8n8k4.f64 (the only tensor-core instruction for binary64 on this
// architecture; tcgen05 has no fp64 kind).  One warp instruction performs 256 FMAs, so
// the shared-memory and issue traffic that limits the DFMA kernel (dgemm_fma.cuh)
// becomes negligible.  Macro-tile 128 x 64 x 8, 8 warps in a 4 x 2 grid, warp tile
// 32 x 32 = 4 x 4 m8n8 accumulators (32 doubles per thread); operands staged through
// double-buffered shared memory [k][rows + 4] (the +4 makes the fragment loads conflict
// free), guarded loads with zero-filled tails, all four transpose modes, any leading
// dimensions.  The write rule is the reference's (src/gemm/ref/Kernels.cpp:87).
// Counterpart of the reference's fp64 kernels (e.g. the 128x64 hand kernel
// src/gemm/assembly/naive_gemm_kernel_MT128x064x08_TT08_04_STT04_04_WG16_16_01.s).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "dgemm_fma.cuh"  // DgemmParams
#include "raster.h"

namespace mmbo {

constexpr int kDmBM = 128, kDmBN = 64, kDmBK = 8, kDmThreads = 256;

template <int ROWS, bool CONTIG_ROW>
struct DmSlab {
  static constexpr int kElems = ROWS * kDmBK / kDmThreads;
  static constexpr int kPitch = ROWS + 4;
  __device__ __forceinline__ static void load(double (&reg)[kElems], const double* __restrict__ base, uint32_t ld,
                                              uint32_t row0, uint32_t l0, uint32_t row_end, uint32_t l_end, int tid) {
#pragma unroll
    for (int e = 0; e < kElems; ++e) {
      const int idx = tid + e * kDmThreads;
      const uint32_t row = CONTIG_ROW ? idx % ROWS : idx / kDmBK;
      const uint32_t l = CONTIG_ROW ? idx / ROWS : idx % kDmBK;
      double x = 0.0;
      if (row0 + row < row_end && l0 + l < l_end) {
        const size_t off = CONTIG_ROW ? (size_t)(row0 + row) + (size_t)(l0 + l) * ld
                                      : (size_t)(l0 + l) + (size_t)(row0 + row) * ld;
        x = __ldg(base + off);
      }
      reg[e] = x;
    }
  }
  __device__ __forceinline__ static void store(const double (&reg)[kElems], double* __restrict__ tile, int tid) {
#pragma unroll
    for (int e = 0; e < kElems; ++e) {
      const int idx = tid + e * kDmThreads;
      const int row = CONTIG_ROW ? idx % ROWS : idx / kDmBK;
      const int l = CONTIG_ROW ? idx / ROWS : idx % kDmBK;
      tile[l * kPitch + row] = reg[e];
    }
  }
};

__device__ __forceinline__ void dmma_m8n8k4(double (&c)[2], double a, double b) {
  asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0, %1}, {%2}, {%3}, {%0, %1};"
               : "+d"(c[0]), "+d"(c[1])
               : "d"(a), "d"(b));
}

template <bool TRANS_A, bool TRANS_B>
__global__ void __launch_bounds__(kDmThreads, 2)
dgemm_dmma_kernel(const double* __restrict__ A, const double* __restrict__ B, double* __restrict__ C,
                  const DgemmParams p) {
  using LA = DmSlab<kDmBM, !TRANS_A>;
  using LB = DmSlab<kDmBN, TRANS_B>;
  __shared__ __align__(16) double sA[2][kDmBK * LA::kPitch];
  __shared__ __align__(16) double sB[2][kDmBK * LB::kPitch];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gid = lane >> 2, tig = lane & 3;      // fragment coordinates of m8n8k4
  const int wm = (warp & 3) * 32, wn = (warp >> 2) * 32;  // warp tile origin inside the block tile
  A += (size_t)blockIdx.z * p.batch_a;  // problem blockIdx.z of a strided batch
  B += (size_t)blockIdx.z * p.batch_b;
  C += (size_t)blockIdx.z * p.batch_c;

  uint32_t tile_m, tile_n;
  mmbo_wgm_remap(blockIdx.x, blockIdx.y, gridDim.x, gridDim.y, p.wgm, &tile_m, &tile_n);
  const uint32_t m0 = tile_m * kDmBM, n0 = tile_n * kDmBN;

  double acc[4][4][2];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;

  double ra[LA::kElems], rb[LB::kElems];
  const uint32_t num_kb = (p.k + kDmBK - 1) / kDmBK;
  LA::load(ra, A, p.lda, m0, 0, p.m, p.k, tid);
  LB::load(rb, B, p.ldb, n0, 0, p.n, p.k, tid);
  LA::store(ra, sA[0], tid);
  LB::store(rb, sB[0], tid);
  __syncthreads();

  for (uint32_t kb = 0; kb < num_kb; ++kb) {
    const int cur = kb & 1;
    if (kb + 1 < num_kb) {
      LA::load(ra, A, p.lda, m0, (kb + 1) * kDmBK, p.m, p.k, tid);
      LB::load(rb, B, p.ldb, n0, (kb + 1) * kDmBK, p.n, p.k, tid);
    }
    const double* __restrict__ a_s = sA[cur];
    const double* __restrict__ b_s = sB[cur];
#pragma unroll
    for (int k4 = 0; k4 < kDmBK; k4 += 4) {
      double fa[4], fb[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) fa[i] = a_s[(k4 + tig) * LA::kPitch + wm + 8 * i + gid];  // A[m = gid][k = tig]
#pragma unroll
      for (int j = 0; j < 4; ++j) fb[j] = b_s[(k4 + tig) * LB::kPitch + wn + 8 * j + gid];  // B[k = tig][n = gid]
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) dmma_m8n8k4(acc[i][j], fa[i], fb[j]);
    }
    if (kb + 1 < num_kb) {
      LA::store(ra, sA[cur ^ 1], tid);
      LB::store(rb, sB[cur ^ 1], tid);
    }
    __syncthreads();
  }

  // accumulator (i, j): C[m = gid][n = 2*tig + {0, 1}] of the 8 x 8 tile at (wm + 8i, wn + 8j)
  const double alpha = p.alpha, beta = p.beta;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t mi = m0 + wm + 8 * i + gid;
    if (mi >= p.m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const uint32_t nj = n0 + wn + 8 * j + 2 * tig + e;
        if (nj >= p.n) continue;
        double* cp = C + (size_t)mi + (size_t)nj * p.ldc;
        double r = alpha * acc[i][j][e];
        if (beta != 0.0) r = fma(beta, *cp, r);
        *cp = r;
      }
  }
}

}  // namespace mmbo
