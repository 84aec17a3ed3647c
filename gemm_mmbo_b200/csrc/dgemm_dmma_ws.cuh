// DGEMM on the fp64 tensor path, warp-specialised and persistent.
//
// The fp64 tensor pipe (mma.sync.m8n8k4.f64, 256 FMAs per warp instruction) is shared with
// nothing else a GEMM needs, so the kernel is arranged so that the four warps that issue it
// do nothing but load fragments from shared memory and multiply:
//   * a producer warpgroup (four warps, 48 registers each after setmaxnreg) fills a ring of
//     kWsStages operand slabs (depth 16) and never computes.  Where an operand's tile rows are
//     contiguous in memory and 16-byte aligned (op(A) of the N modes, op(B) of the T modes:
//     both operands of the reference's dgemm_NT) each k-row of the slab is one bulk
//     asynchronous copy (cp.async.bulk, the 1-D form of TMA) into a padded row, issued by the
//     first producer warp; otherwise (K-contiguous operands, ragged edges, the K tail, odd
//     leading dimensions) the 128 producer lanes issue 8-byte cp.async copies that transpose
//     on the way in and zero-fill outside the matrix.  Either way completion is counted on the
//     slab's "full" mbarrier; consumers hand slabs back through "empty" mbarriers.  There is
//     no block-wide barrier in the main loop;
//   * a consumer warpgroup (four warps, 208 registers each), every warp owning a 64 x 32
//     piece of the 128 x 64 tile (64 accumulator doubles per thread, 12 fragment loads per
//     32 tensor instructions); a second instantiation with 64 x 64 tiles (32 x 32 per warp)
//     serves problems that have too few 128-row tiles to fill the machine.  The registers taken from the producers let the epilogue keep
//     32 values of C in flight per thread, so that reading C costs two memory round trips per
//     tile instead of one per value;
//   * two CTAs per SM, each walking tiles of the remapped order (raster.h) with a stride of
//     the grid: while one CTA's consumers read-modify-write C, the other CTA's keep the pipe
//     busy, and the producers are already filling slabs of the next tile.
// Every wait is bounded (ptx.cuh): on a time-out the device status word is set and all
// roles leave after the producers have waited for their copies in flight.
// The write rule is the reference's (src/gemm/ref/Kernels.cpp:87); the kernel is the
// counterpart of its 128x64 hand kernel for the HPL update
// (src/gemm/assembly/naive_gemm_kernel_MT128x064x08_TT08_04_STT04_04_WG16_16_01.s).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "dgemm_dmma.cuh"  // dmma_m8n8k4, DgemmParams
#include "ptx.cuh"
#include "raster.h"

namespace mmbo {

// Tile rows BM = 128 (warp tile 64 x 32) or 64 (warp tile 32 x 32, for problems with too few 128-row tiles
// to fill the machine twice).
constexpr int kWsBN = 64, kWsBK = 16, kWsStages = 4;
constexpr int kWsConsumers = 4, kWsProducers = 4, kWsThreads = (kWsConsumers + kWsProducers) * 32;
constexpr int kWsPitchB = kWsBN + 4;  // doubles; +4 keeps fragment loads conflict-free
constexpr int kWsSlabB = kWsBK * kWsPitchB;
template <int BM>
struct WsTile {
  static constexpr int kPitchA = BM + 4;
  static constexpr int kSlabA = kWsBK * kPitchA;
  static constexpr size_t kSmemBytes = (size_t)kWsStages * (kSlabA + kWsSlabB) * sizeof(double);
  static constexpr int kFragM = BM / 16;  // m8 fragments per consumer warp (two warps along m)
};
// arrivals that complete a slab: one cp.async arrival per producer lane + the expect_tx arrival
constexpr uint32_t kWsFullCount = kWsProducers * 32 + 1;

__device__ __forceinline__ void ws_cp_async_8(uint32_t smem_dst, const void* gmem_src, bool valid) {
  const uint32_t bytes = valid ? 8u : 0u;  // source size 0: the slot is zero-filled
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(smem_dst), "l"(gmem_src), "r"(bytes) : "memory");
}
// The barrier receives one arrival once all cp.async copies this thread issued so far have landed.
__device__ __forceinline__ void ws_cp_async_arrive(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void ws_cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void ws_bulk_row(uint32_t smem_dst, const void* gmem_src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_dst), "l"(gmem_src), "r"(bytes), "r"(bar) : "memory");
}

// Element-wise slab fill, this producer warp's share (1 / NP) of it.  CONTIG_ROW: the tile-row index
// (m or n) is the contiguous one in memory.  One 64-bit add per copy; GUARD adds the bounds
// checks (source size 0 zero-fills) and is only instantiated for edge tiles and the K tail.
template <int ROWS, bool CONTIG_ROW, bool GUARD, int NP>
__device__ __forceinline__ void ws_fill_elements(uint32_t slab, const double* __restrict__ base, uint32_t ld,
                                                 uint32_t row0, uint32_t l0, uint32_t row_end, uint32_t l_end,
                                                 int lane, int pw) {
  constexpr int kPitch = ROWS + 4;
  if constexpr (CONTIG_ROW) {  // a warp copy covers 32 consecutive rows of one k-row; warp pw takes 16 / NP k-rows
    constexpr int kRowsPerWarp = kWsBK / NP;
    const uint32_t lw = pw * kRowsPerWarp;
    const double* src = base + (size_t)row0 + lane + (size_t)(l0 + lw) * ld;
    const uint32_t dst = slab + (lw * kPitch + lane) * 8u;
#pragma unroll 4
    for (int l = 0; l < kRowsPerWarp; ++l) {
      const bool l_ok = !GUARD || l0 + lw + l < l_end;
#pragma unroll
      for (int c = 0; c < ROWS / 32; ++c) {
        const bool ok = !GUARD || (l_ok && row0 + lane + 32 * c < row_end);
        ws_cp_async_8(dst + (l * kPitch + 32 * c) * 8u, ok ? src + 32 * c : base, ok);
      }
      src += ld;
    }
  } else {  // a warp copy covers 16 consecutive k of two rows and transposes on the way in; warp pw takes 1 / NP of the rows
    constexpr int kPairs = ROWS / 2 / NP;
    const uint32_t l = lane & 15, r = (lane >> 4) + 2 * kPairs * pw;
    const bool l_ok = !GUARD || l0 + l < l_end;
    const double* src = base + (size_t)(l0 + l) + (size_t)(row0 + r) * ld;
    const uint32_t dst = slab + (l * kPitch + r) * 8u;
    const size_t step = 2 * (size_t)ld;
#pragma unroll 8
    for (int e = 0; e < kPairs; ++e) {
      const bool ok = !GUARD || (l_ok && row0 + r + 2 * e < row_end);
      ws_cp_async_8(dst + e * 16u, ok ? src : base, ok);
      src += step;
    }
  }
}

template <bool TRANS_A, bool TRANS_B, int BM>
__global__ void __launch_bounds__(kWsThreads, 2)
dgemm_dmma_ws_kernel(const double* __restrict__ A, const double* __restrict__ B, double* __restrict__ C,
                     const DgemmParams p) {
  using T = WsTile<BM>;
  constexpr int kWsBM = BM, kWsPitchA = T::kPitchA, kWsSlabA = T::kSlabA, kFragM = T::kFragM;
  static_assert(BM == 128 || BM == 64, "two consumer warps along m, 64 or 32 rows each");
  extern __shared__ __align__(128) double ws_smem[];
  __shared__ __align__(8) uint64_t full_bar[kWsStages], empty_bar[kWsStages];
  __shared__ uint32_t abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t smem_a = smem_u32(ws_smem);
  const uint32_t smem_b = smem_a + kWsStages * kWsSlabA * 8u;
  // When both operands qualify for bulk copies the first producer warp feeds the ring alone
  // (its lanes also cover the few edge and K-tail slabs) and the other three leave at once,
  // so that no idle warp polls barriers next to the consumers.
  const bool solo = !TRANS_A && TRANS_B && ((reinterpret_cast<uintptr_t>(A) & 15u) == 0) && (p.lda & 1u) == 0 &&
                    ((reinterpret_cast<uintptr_t>(B) & 15u) == 0) && (p.ldb & 1u) == 0;
  if (tid == 0) {
    abort_flag = 0;
    for (int s = 0; s < kWsStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), solo ? 33u : kWsFullCount);
      mbar_init(smem_u32(&empty_bar[s]), kWsConsumers);
    }
    fence_mbar_init();
  }
  __syncthreads();

  const uint32_t tiles_m = (p.m + kWsBM - 1) / kWsBM, tiles_n = (p.n + kWsBN - 1) / kWsBN;
  const uint32_t num_tiles = tiles_m * tiles_n;
  const uint32_t num_kb = (p.k + kWsBK - 1) / kWsBK;
  uint32_t stage = 0, phase = 0;

  if (warp >= kWsConsumers) {
    // ----------------------------------------------------------------- producers ----
    asm volatile("setmaxnreg.dec.sync.aligned.u32 48;");
    const int pw = warp - kWsConsumers;
    if (solo && pw != 0) return;
    const bool a_rows_bulk = !TRANS_A && ((reinterpret_cast<uintptr_t>(A) & 15u) == 0) && (p.lda & 1u) == 0;
    const bool b_rows_bulk = TRANS_B && ((reinterpret_cast<uintptr_t>(B) & 15u) == 0) && (p.ldb & 1u) == 0;
    // the epilogue's C lines are requested from L2 this many slabs before the tile's last one
    const uint32_t c_prefetch_kb = num_kb > 24u ? num_kb - 24u : 0u;
    uint32_t issued = 0;
    bool ok = true;
    for (uint32_t tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      uint32_t tile_m, tile_n;
      mmbo_tile_from_serial(tile, tiles_m, tiles_n, p.wgm, &tile_m, &tile_n);
      const uint32_t m0 = tile_m * kWsBM, n0 = tile_n * kWsBN;
      const bool a_inside = m0 + kWsBM <= p.m, b_inside = n0 + kWsBN <= p.n;
      for (uint32_t kb = 0; kb < num_kb; ++kb) {
        if (p.beta != 0.0 && kb == c_prefetch_kb) {
          // ask L2 for this tile's C lines: 64 columns of up to 1 KB, 16 columns per producer warp
          const uint32_t rows = p.m - m0 < (uint32_t)kWsBM ? p.m - m0 : (uint32_t)kWsBM;
          // (bulk prefetch, the 1-D form of the TMA prefetch, where the column pieces are 16-byte
          // aligned: one request per column; otherwise one prefetch per 128-byte line)
          const bool c_bulk = ((reinterpret_cast<uintptr_t>(C) & 15u) == 0) && (p.ldc & 1u) == 0 && (rows & 1u) == 0;
          const uint32_t c_first = solo ? 0u : 16u * pw, c_last = solo ? (uint32_t)kWsBN : 16u * pw + 16u;
          if (c_bulk) {
            for (uint32_t c = c_first + lane; c < c_last; c += 32) {
              const uint32_t col = n0 + c;
              if (col < p.n)
                asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(C + (size_t)col * p.ldc + m0), "r"(rows * 8u)
                             : "memory");
            }
          } else {
            for (uint32_t c = c_first; c < c_last; c += 16) {
              const uint32_t col = n0 + c + (lane >> 1);
              if (col < p.n) {
                const double* c_col = C + (size_t)col * p.ldc + m0;
                for (uint32_t r = (lane & 1) * 16; r < rows; r += 32) asm volatile("prefetch.global.L2 [%0];" ::"l"(c_col + r));
                if (lane & 1) asm volatile("prefetch.global.L2 [%0];" ::"l"(c_col + rows - 1));
              }
            }
          }
        }
        const uint32_t full = smem_u32(&full_bar[stage]);
        if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, &abort_flag, kFaultWaitEmpty, stage)) {
          ok = false;
          break;
        }
        const uint32_t l0 = kb * kWsBK;
        const bool whole = l0 + kWsBK <= p.k;
        const bool a_bulk = a_rows_bulk && a_inside && whole, b_bulk = b_rows_bulk && b_inside && whole;
        const uint32_t slab_a = smem_a + stage * kWsSlabA * 8u, slab_b = smem_b + stage * kWsSlabB * 8u;
        if (pw == 0) {
          if (lane == 0) {
            const uint32_t tx = (a_bulk ? kWsBK * kWsBM * 8u : 0u) + (b_bulk ? kWsBK * kWsBN * 8u : 0u);
            if (tx) mbar_expect_tx(full, tx);
            else mbar_arrive(full);
          }
          __syncwarp();
          if (a_bulk && lane < kWsBK)
            ws_bulk_row(slab_a + lane * kWsPitchA * 8u, A + (size_t)m0 + (size_t)(l0 + lane) * p.lda, kWsBM * 8u, full);
          if (b_bulk && lane >= 32 - kWsBK)
            ws_bulk_row(slab_b + (lane - (32 - kWsBK)) * kWsPitchB * 8u,
                        B + (size_t)n0 + (size_t)(l0 + lane - (32 - kWsBK)) * p.ldb, kWsBN * 8u, full);
        }
        if (!a_bulk) {
          if (solo) ws_fill_elements<kWsBM, !TRANS_A, true, 1>(slab_a, A, p.lda, m0, l0, p.m, p.k, lane, 0);
          else if (whole && a_inside) ws_fill_elements<kWsBM, !TRANS_A, false, kWsProducers>(slab_a, A, p.lda, m0, l0, p.m, p.k, lane, pw);
          else ws_fill_elements<kWsBM, !TRANS_A, true, kWsProducers>(slab_a, A, p.lda, m0, l0, p.m, p.k, lane, pw);
        }
        if (!b_bulk) {
          if (solo) ws_fill_elements<kWsBN, TRANS_B, true, 1>(slab_b, B, p.ldb, n0, l0, p.n, p.k, lane, 0);
          else if (whole && b_inside) ws_fill_elements<kWsBN, TRANS_B, false, kWsProducers>(slab_b, B, p.ldb, n0, l0, p.n, p.k, lane, pw);
          else ws_fill_elements<kWsBN, TRANS_B, true, kWsProducers>(slab_b, B, p.ldb, n0, l0, p.n, p.k, lane, pw);
        }
        ws_cp_async_arrive(full);
        ++issued;
        if (++stage == kWsStages) { stage = 0; phase ^= 1u; }
      }
    }
    if (!ok || abort_flag) {
      // Leave only after the copies in flight have landed: the element copies of this warp, and
      // the bulk copies of the slabs issued last (a short bounded wait on their full barriers).
      ws_cp_async_wait_all();
      const uint32_t pending = issued < (uint32_t)kWsStages ? issued : (uint32_t)kWsStages;
      for (uint32_t i = 0; pw == 0 && i < pending; ++i) {
        stage = stage == 0 ? kWsStages - 1 : stage - 1;
        if (stage == kWsStages - 1) phase ^= 1u;
        const uint64_t t0 = global_timer_ns();
        while (!mbar_try_wait(smem_u32(&full_bar[stage]), phase) && global_timer_ns() - t0 < MMBO_DRAIN_LIMIT_NS) {
        }
      }
    }
    return;
  }

  // -------------------------------------------------------------------- consumers ----
  asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
  const int gid = lane >> 2, tig = lane & 3;                // fragment coordinates of m8n8k4
  const int wm = (warp & 1) * (BM / 2), wn = (warp >> 1) * 32;  // this warp's (BM / 2) x 32 piece of the tile
  const double alpha = p.alpha, beta = p.beta;
  for (uint32_t tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
    uint32_t tile_m, tile_n;
    mmbo_tile_from_serial(tile, tiles_m, tiles_n, p.wgm, &tile_m, &tile_n);
    const uint32_t m0 = tile_m * kWsBM, n0 = tile_n * kWsBN;
    double acc[kFragM][4][2];
#pragma unroll
    for (int i = 0; i < kFragM; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;

    for (uint32_t kb = 0; kb < num_kb; ++kb) {
      if (!mbar_wait(smem_u32(&full_bar[stage]), phase, &abort_flag, kFaultWaitFull, stage)) return;
      const double* __restrict__ a_s = ws_smem + stage * kWsSlabA + wm + gid;
      const double* __restrict__ b_s = ws_smem + kWsStages * kWsSlabA + stage * kWsSlabB + wn + gid;
#pragma unroll
      for (int k4 = 0; k4 < kWsBK; k4 += 4) {
        double fa[kFragM], fb[4];
#pragma unroll
        for (int i = 0; i < kFragM; ++i) fa[i] = a_s[(k4 + tig) * kWsPitchA + 8 * i];  // A[m = gid][k = tig]
#pragma unroll
        for (int j = 0; j < 4; ++j) fb[j] = b_s[(k4 + tig) * kWsPitchB + 8 * j];  // B[k = tig][n = gid]
#pragma unroll
        for (int i = 0; i < kFragM; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) dmma_m8n8k4(acc[i][j], fa[i], fb[j]);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&empty_bar[stage]));
      if (++stage == kWsStages) { stage = 0; phase ^= 1u; }
    }

    // accumulator (i, j): C[m = gid][n = 2*tig + {0, 1}] of the 8 x 8 block at (wm + 8i, wn + 8j).
    // C is read 32 values per thread at a time (four columns x eight row blocks, one asm block
    // so that the loads are issued back to back) and the tile is done in two such rounds.
    if ((p.diag & 1u) == 0u) {
      const uint32_t row = m0 + wm + gid;
      const uint32_t rows_left = p.m > row ? p.m - row : 0u;  // row block i is inside the matrix iff 8i < rows_left
#pragma unroll
      for (int jh = 0; jh < 2; ++jh) {
        double old[4][kFragM];
        double* c_col[4];
        bool col_ok[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {  // q = 2 * (j & 1) + e
          const uint32_t col = n0 + wn + 8 * (2 * jh + (q >> 1)) + 2 * tig + (q & 1);
          col_ok[q] = col < p.n;
          c_col[q] = C + (size_t)col * p.ldc + row;
        }
        if (beta != 0.0) {
#pragma unroll
          for (int q = 0; q < 4; ++q)
#pragma unroll
            for (int i = 0; i < kFragM; ++i) old[q][i] = (col_ok[q] && 8u * i < rows_left) ? __ldcg(c_col[q] + 8 * i) : 0.0;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
          for (int i = 0; i < kFragM; ++i) {
            if (!col_ok[q] || 8u * i >= rows_left) continue;
            double r = alpha * acc[i][2 * jh + (q >> 1)][q & 1];
            if (beta != 0.0) r = fma(beta, old[q][i], r);
            c_col[q][8 * i] = r;
          }
      }
    }
  }
}

}  // namespace mmbo
