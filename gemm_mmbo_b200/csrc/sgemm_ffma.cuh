// SGEMM on the CUDA cores (FFMA):  C = alpha * op(A) * op(B) + beta * C, fp32 throughout,
// column-major, any leading dimensions, all four transpose modes, ragged edges.
//
// This is the B200 counterpart of the reference's general (Tensile) path
// (src/gemm/ref/Kernels.cpp:153-1123): a macro-tile BM x BN per thread block, DepthU =
// BK, a TTM x TTN micro-tile per thread, operands staged through double-buffered shared
// memory, zero-filled tails instead of the reference's pointer shifting, and the
// reference's write rule (Kernels.cpp:87: beta == 0 never reads C).  Differences that
// matter on this hardware: 128-bit shared and global accesses wherever alignment
// allows (run-time check, scalar guarded path otherwise), register prefetch of the
// next slab during the FFMA burst, and micro-tiles split into 4-wide halves 64
// elements apart so that a warp's shared-memory reads are conflict-free and its C
// stores cover 256 contiguous bytes.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"
#include "raster.h"

namespace mmbo {

struct SgemmParams {
  uint32_t m, n, k;
  uint32_t lda, ldb, ldc;
  float alpha, beta;
  uint32_t wgm;
  uint32_t vec_a, vec_b, vec_c;  // 1 when 128-bit accesses to that operand are legal
  // strided batch (the reference's kernel takes the problem index from the third grid dimension,
  // src/gemm/ref/Kernels.cpp:254): elements between consecutive problems' A, B, C
  unsigned long long batch_a, batch_b, batch_c;
};

// Loads a (ROWS x BK) slab of an operand into registers.  "row" is the M (or N) index
// inside the tile, "l" the K index.  CONTIG_ROW = the operand's row index is the
// contiguous one in memory (A not transposed / B transposed).
template <int ROWS, int BK, int THREADS, bool CONTIG_ROW>
struct SlabLoader {
  static constexpr int kElems = ROWS * BK / THREADS;  // per thread
  static constexpr int kVecs = kElems / 4;
  static_assert(kElems % 4 == 0, "slab must split into float4 per thread");

  __device__ __forceinline__ static void load(float (&reg)[kElems], const float* __restrict__ base,
                                              uint32_t ld, uint32_t row0, uint32_t l0,
                                              uint32_t row_end, uint32_t l_end, bool vec, int tid) {
    if (vec) {
#pragma unroll
      for (int v = 0; v < kVecs; ++v) {
        const int idx = tid + v * THREADS;
        uint32_t row, l;
        if (CONTIG_ROW) {
          l = idx / (ROWS / 4);
          row = (idx % (ROWS / 4)) * 4;
        } else {
          row = idx / (BK / 4);
          l = (idx % (BK / 4)) * 4;
        }
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row0 + row < row_end && l0 + l < l_end) {
          const size_t off = CONTIG_ROW ? (size_t)(row0 + row) + (size_t)(l0 + l) * ld
                                        : (size_t)(l0 + l) + (size_t)(row0 + row) * ld;
          x = __ldg(reinterpret_cast<const float4*>(base + off));
        }
        reg[4 * v + 0] = x.x;
        reg[4 * v + 1] = x.y;
        reg[4 * v + 2] = x.z;
        reg[4 * v + 3] = x.w;
      }
    } else {
#pragma unroll
      for (int e = 0; e < kElems; ++e) {
        // Same element-to-thread assignment as the vector path, one element at a time.
        const int idx = tid + (e / 4) * THREADS;
        uint32_t row, l;
        if (CONTIG_ROW) {
          l = idx / (ROWS / 4);
          row = (idx % (ROWS / 4)) * 4 + (e % 4);
        } else {
          row = idx / (BK / 4);
          l = (idx % (BK / 4)) * 4 + (e % 4);
        }
        float x = 0.f;
        if (row0 + row < row_end && l0 + l < l_end) {
          const size_t off = CONTIG_ROW ? (size_t)(row0 + row) + (size_t)(l0 + l) * ld
                                        : (size_t)(l0 + l) + (size_t)(row0 + row) * ld;
          x = __ldg(base + off);
        }
        reg[e] = x;
      }
    }
  }

  // Shared tile layout: [BK][ROWS + 4] floats (row index contiguous).
  __device__ __forceinline__ static void store(const float (&reg)[kElems], float* __restrict__ tile,
                                               int tid) {
    constexpr int kPitch = ROWS + 4;
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
      const int idx = tid + v * THREADS;
      if (CONTIG_ROW) {
        const int l = idx / (ROWS / 4);
        const int row = (idx % (ROWS / 4)) * 4;
        *reinterpret_cast<float4*>(tile + l * kPitch + row) =
            make_float4(reg[4 * v], reg[4 * v + 1], reg[4 * v + 2], reg[4 * v + 3]);
      } else {
        const int row = idx / (BK / 4);
        const int l = (idx % (BK / 4)) * 4;
#pragma unroll
        for (int e = 0; e < 4; ++e) tile[(l + e) * kPitch + row] = reg[4 * v + e];
      }
    }
  }
};

template <int BM, int BN, int BK, int TTM, int TTN, bool TRANS_A, bool TRANS_B>
__global__ void __launch_bounds__((BM / TTM) * (BN / TTN), (TTM * TTN >= 64 ? 2 : 3))
sgemm_ffma_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C,
                  const SgemmParams p) {
  constexpr int THREADS = (BM / TTM) * (BN / TTN);
  constexpr int TX = BM / TTM;  // threads along M (lanes vary along M first)
  constexpr int HM = TTM / 4;   // 4-wide pieces of the micro-tile along M ...
  constexpr int HN = TTN / 4;   // ... and along N
  constexpr int PA = BM + 4, PB = BN + 4;
  static_assert(TTM % 4 == 0 && TTN % 4 == 0, "micro-tile is built from 4-wide pieces");

  using LoadA = SlabLoader<BM, BK, THREADS, !TRANS_A>;
  using LoadB = SlabLoader<BN, BK, THREADS, TRANS_B>;

  __shared__ __align__(16) float sA[2][BK * PA];
  __shared__ __align__(16) float sB[2][BK * PB];

  const int tid = threadIdx.x;
  const int tx = tid % TX, ty = tid / TX;
  A += (size_t)blockIdx.z * p.batch_a;  // problem blockIdx.z of a strided batch
  B += (size_t)blockIdx.z * p.batch_b;
  C += (size_t)blockIdx.z * p.batch_c;

  uint32_t tile_m, tile_n;
  mmbo_wgm_remap(blockIdx.x, blockIdx.y, gridDim.x, gridDim.y, p.wgm, &tile_m, &tile_n);
  const uint32_t m0 = tile_m * BM, n0 = tile_n * BN;

  // Accumulators as packed pairs along m: one fma.rn.f32x2 updates two of them, so the 64
  // FMAs of a k step take 32 issue slots and leave room for the loads and the loop.
  uint64_t acc2[TTN][TTM / 2];
#pragma unroll
  for (int j = 0; j < TTN; ++j)
#pragma unroll
    for (int i = 0; i < TTM / 2; ++i) acc2[j][i] = 0ull;

  float ra[LoadA::kElems], rb[LoadB::kElems];
  const uint32_t num_kb = (p.k + BK - 1) / BK;

  LoadA::load(ra, A, p.lda, m0, 0, p.m, p.k, p.vec_a != 0, tid);
  LoadB::load(rb, B, p.ldb, n0, 0, p.n, p.k, p.vec_b != 0, tid);
  LoadA::store(ra, sA[0], tid);
  LoadB::store(rb, sB[0], tid);
  __syncthreads();

  for (uint32_t kb = 0; kb < num_kb; ++kb) {
    const int cur = kb & 1;
    if (kb + 1 < num_kb) {
      LoadA::load(ra, A, p.lda, m0, (kb + 1) * BK, p.m, p.k, p.vec_a != 0, tid);
      LoadB::load(rb, B, p.ldb, n0, (kb + 1) * BK, p.n, p.k, p.vec_b != 0, tid);
    }
    const float* __restrict__ a_s = sA[cur];
    const float* __restrict__ b_s = sB[cur];
#pragma unroll
    for (int l = 0; l < BK; ++l) {
      uint64_t fa2[TTM / 2];
      float fb[TTN];
#pragma unroll
      for (int h = 0; h < HM; ++h) {
        const uint4 x = *reinterpret_cast<const uint4*>(a_s + l * PA + h * (BM / HM) + tx * 4);
        fa2[2 * h] = pack_f32x2(x.x, x.y);
        fa2[2 * h + 1] = pack_f32x2(x.z, x.w);
      }
#pragma unroll
      for (int h = 0; h < HN; ++h) {
        const float4 x = *reinterpret_cast<const float4*>(b_s + l * PB + h * (BN / HN) + ty * 4);
        fb[4 * h] = x.x; fb[4 * h + 1] = x.y; fb[4 * h + 2] = x.z; fb[4 * h + 3] = x.w;
      }
#pragma unroll
      for (int j = 0; j < TTN; ++j) {
        const uint64_t bb = pack_f32x2(__float_as_uint(fb[j]), __float_as_uint(fb[j]));
#pragma unroll
        for (int i = 0; i < TTM / 2; ++i) acc2[j][i] = fma_f32x2(fa2[i], bb, acc2[j][i]);
      }
    }
    if (kb + 1 < num_kb) {
      LoadA::store(ra, sA[cur ^ 1], tid);
      LoadB::store(rb, sB[cur ^ 1], tid);
    }
    __syncthreads();
  }

  // Write-back: C = beta != 0 ? alpha*acc + beta*C : alpha*acc.
  const float alpha = p.alpha, beta = p.beta;
  const bool use_c = beta != 0.f;
  float acc[TTN][TTM];
#pragma unroll
  for (int j = 0; j < TTN; ++j)
#pragma unroll
    for (int i = 0; i < TTM / 2; ++i) {
      acc[j][2 * i] = __uint_as_float((uint32_t)(acc2[j][i] & 0xffffffffull));
      acc[j][2 * i + 1] = __uint_as_float((uint32_t)(acc2[j][i] >> 32));
    }
#pragma unroll
  for (int hn = 0; hn < HN; ++hn)
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const uint32_t j = n0 + hn * (BN / HN) + ty * 4 + jj;
      if (j >= p.n) continue;
#pragma unroll
      for (int hm = 0; hm < HM; ++hm) {
        const uint32_t i = m0 + hm * (BM / HM) + tx * 4;
        if (i >= p.m) continue;
        float* cp = C + (size_t)i + (size_t)j * p.ldc;
        const float* a4 = &acc[hn * 4 + jj][hm * 4];
        if (p.vec_c && i + 3 < p.m) {
          float4 o = make_float4(alpha * a4[0], alpha * a4[1], alpha * a4[2], alpha * a4[3]);
          if (use_c) {
            const float4 c4 = *reinterpret_cast<const float4*>(cp);
            o.x = fmaf(beta, c4.x, o.x);
            o.y = fmaf(beta, c4.y, o.y);
            o.z = fmaf(beta, c4.z, o.z);
            o.w = fmaf(beta, c4.w, o.w);
          }
          *reinterpret_cast<float4*>(cp) = o;
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            if (i + e < p.m) {
              float o = alpha * a4[e];
              if (use_c) o = fmaf(beta, cp[e], o);
              cp[e] = o;
            }
          }
        }
      }
    }
}

}  // namespace mmbo
