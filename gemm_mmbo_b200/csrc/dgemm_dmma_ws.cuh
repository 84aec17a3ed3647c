// DGEMM on the fp64 tensor path, warp-specialised and persistent.
//
// The fp64 tensor pipe (mma.sync.m8n8k4.f64, 256 FMAs per warp instruction) is shared with
// nothing else a GEMM needs, so the kernel is arranged so that the four warps that issue it
// do nothing but load fragments from shared memory and multiply:
//   * a producer warpgroup (four warps, 48 registers each after setmaxnreg) fills a ring of
//     operand slabs (depth 16) and never computes.  An operand with a 16-byte aligned base and
//     an even leading dimension comes in through TMA, one cp.async.bulk.tensor per slab: the
//     box is four elements wider than the tile along the contiguous dimension, which lays the
//     slab out with the padded pitch that keeps the fragment loads free of bank conflicts
//     ([k][rows + 4] when the tile rows are contiguous in memory, [row][16 + 4] when k is), and
//     edges and the K tail are zero-filled by the copy engine.  When both operands qualify one
//     producer warp feeds alone and the other three leave.  Operands TMA cannot address (odd
//     leading dimension, base off a 16-byte boundary) are filled by the 128 producer lanes with
//     8-byte cp.async copies, zero-filling outside the matrix.  Either way completion is
//     counted on the slab's "full" mbarrier; consumers hand slabs back through "empty"
//     mbarriers.  There is no block-wide barrier in the main loop;
//   * a consumer warpgroup (four warps, 208 registers each), every warp owning a 64 x 32
//     piece of the 128 x 64 tile (64 accumulator doubles per thread, 12 fragment loads per
//     32 tensor instructions); a second instantiation with 64 x 64 tiles (32 x 32 per warp)
//     exists as a table row.  The registers taken from the producers let the epilogue keep
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

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "dgemm_dmma.cuh"  // dmma_m8n8k4, DgemmParams
#include "ptx.cuh"
#include "raster.h"
#include "stream_k.cuh"

namespace mmbo {

constexpr int kWsBN = 64, kWsBK = 16;
constexpr int kWsConsumers = 4, kWsProducers = 4, kWsThreads = (kWsConsumers + kWsProducers) * 32;
constexpr int kWsPad = 4;  // extra elements per shared-memory row (and per TMA box row)

// One operand slab in shared memory.  KMAJOR: k is the contiguous index in memory, the slab
// is [row][16 + 4]; otherwise the tile-row index (m or n) is, and the slab is [k][ROWS + 4].
// Either pitch makes the 16 fragment loads of a half-warp hit 16 distinct bank pairs.
template <int ROWS, bool KMAJOR>
struct WsSlab {
  static constexpr int kPitch = (KMAJOR ? kWsBK : ROWS) + kWsPad;
  static constexpr int kLines = KMAJOR ? ROWS : kWsBK;
  static constexpr int kDoubles = kLines * kPitch;
  static constexpr uint32_t kBytes = kDoubles * 8u;  // = bytes one TMA box delivers
  __host__ __device__ static constexpr int at(int row, int l) { return KMAJOR ? row * kPitch + l : l * kPitch + row; }
};

template <int BM, bool A_KMAJOR, bool B_KMAJOR>
struct WsTile {
  using SA = WsSlab<BM, A_KMAJOR>;
  using SB = WsSlab<kWsBN, B_KMAJOR>;
  static constexpr int kStageDoubles = SA::kDoubles + SB::kDoubles;
  // 64-row tiles leave room for the tile's old C, [col][BM + 4]: the producer brings it in with
  // one TMA box well ahead of the epilogue that needs it, which then reads shared memory
  // instead of waiting for HBM twice.
  static constexpr bool kStageC = BM == 64;
  static constexpr int kCPitch = BM + kWsPad;
  static constexpr int kCDoubles = kStageC ? kWsBN * kCPitch : 0;
  // two CTAs per SM: at most about 115 KB of dynamic shared memory each
  static constexpr int kStages = ((size_t)4 * kStageDoubles + kCDoubles) * 8 + 128 <= 115000 ? 4 : 3;
  static constexpr size_t kSmemBytes = ((size_t)kStages * kStageDoubles + kCDoubles) * sizeof(double) + 128;  // + slack to align the ring
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

// Element-wise slab fill for an operand TMA cannot address, this producer warp's share
// (1 / NP) of it.  One 64-bit add per copy; GUARD adds the bounds checks (source size 0
// zero-fills) and is only instantiated for edge tiles and the K tail.
template <int ROWS, bool KMAJOR, bool GUARD, int NP>
__device__ __forceinline__ void ws_fill_elements(uint32_t slab, const double* __restrict__ base, uint32_t ld,
                                                 uint32_t row0, uint32_t l0, uint32_t row_end, uint32_t l_end,
                                                 int lane, int pw) {
  using S = WsSlab<ROWS, KMAJOR>;
  if constexpr (!KMAJOR) {  // a warp copy covers 32 consecutive rows of one k-row; warp pw takes 16 / NP k-rows
    constexpr int kRowsPerWarp = kWsBK / NP;
    const uint32_t lw = pw * kRowsPerWarp;
    const double* src = base + (size_t)row0 + lane + (size_t)(l0 + lw) * ld;
    const uint32_t dst = slab + (lw * S::kPitch + lane) * 8u;
#pragma unroll 4
    for (int l = 0; l < kRowsPerWarp; ++l) {
      const bool l_ok = !GUARD || l0 + lw + l < l_end;
#pragma unroll
      for (int c = 0; c < ROWS / 32; ++c) {
        const bool ok = !GUARD || (l_ok && row0 + lane + 32 * c < row_end);
        ws_cp_async_8(dst + (l * S::kPitch + 32 * c) * 8u, ok ? src + 32 * c : base, ok);
      }
      src += ld;
    }
  } else {  // a warp copy covers 16 consecutive k of two rows; warp pw takes 1 / NP of the rows
    constexpr int kPairs = ROWS / 2 / NP;
    const uint32_t l = lane & 15, r = (lane >> 4) + 2 * kPairs * pw;
    const bool l_ok = !GUARD || l0 + l < l_end;
    const double* src = base + (size_t)(l0 + l) + (size_t)(row0 + r) * ld;
    const uint32_t dst = slab + (r * S::kPitch + l) * 8u;
    const size_t step = 2 * (size_t)ld;
#pragma unroll 8
    for (int e = 0; e < kPairs; ++e) {
      const bool ok = !GUARD || (l_ok && row0 + r + 2 * e < row_end);
      ws_cp_async_8(dst + e * 2 * S::kPitch * 8u, ok ? src : base, ok);
      src += step;
    }
  }
}

template <bool TRANS_A, bool TRANS_B, int BM, bool SK = false>
__global__ void __launch_bounds__(kWsThreads, 2)
dgemm_dmma_ws_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                     const __grid_constant__ CUtensorMap tmap_c, const double* __restrict__ A, const double* __restrict__ B, double* __restrict__ C,
                     const DgemmParams p, const StreamK sk) {
  constexpr bool A_KMAJOR = TRANS_A, B_KMAJOR = !TRANS_B;  // which index is contiguous in memory
  using T = WsTile<BM, A_KMAJOR, B_KMAJOR>;
  using SA = typename T::SA;
  using SB = typename T::SB;
  constexpr int kStages = T::kStages, kFragM = T::kFragM;
  static_assert(BM == 128 || BM == 64, "two consumer warps along m, 64 or 32 rows each");
  extern __shared__ __align__(16) uint8_t ws_smem_raw[];
  // TMA writes whole boxes to 128-byte aligned shared memory
  double* const ws_smem = reinterpret_cast<double*>(ws_smem_raw + ((128u - (smem_u32(ws_smem_raw) & 127u)) & 127u));
  __shared__ __align__(8) uint64_t full_bar[kStages], empty_bar[kStages];
  __shared__ __align__(8) uint64_t c_full_bar, c_empty_bar;  // the staged C tile (64-row tiles, p.tma_c)
  __shared__ uint32_t abort_flag;
  const bool stage_c = T::kStageC && p.tma_c && p.beta != 0.0;
  double* const c_smem = ws_smem + kStages * T::kStageDoubles;  // [col][BM + 4]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t smem_a = smem_u32(ws_smem);
  const uint32_t smem_b = smem_a + kStages * SA::kBytes;
  // When both operands come in through TMA the first producer warp feeds the ring alone and the
  // other three leave at once, so that no idle warp polls barriers next to the consumers.
  const bool solo = p.tma_a && p.tma_b;
  if (tid == 0) {
    abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), solo ? 33u : kWsFullCount);
      mbar_init(smem_u32(&empty_bar[s]), kWsConsumers);
    }
    mbar_init(smem_u32(&c_full_bar), 1);
    mbar_init(smem_u32(&c_empty_bar), kWsConsumers);
    fence_mbar_init();
  }
  __syncthreads();

  const uint32_t tiles_m = (p.m + BM - 1) / BM, tiles_n = (p.n + kWsBN - 1) / kWsBN;
  const uint32_t tiles_per_problem = tiles_m * tiles_n;
  const uint32_t num_tiles = tiles_per_problem * p.batch;  // strided batch: problem index slowest
  const uint32_t num_kb = (p.k + kWsBK - 1) / kWsBK;
  uint32_t stage = 0, phase = 0;
  const bool batched = p.batch > 1u;  // 3-D tensor maps; single problems keep the 2-D forms
  auto locate = [&](uint32_t tile, uint32_t* tm, uint32_t* tn) -> uint32_t {
    const uint32_t prob = tile / tiles_per_problem;
    mmbo_tile_from_serial(tile - prob * tiles_per_problem, tiles_m, tiles_n, p.wgm, tm, tn);
    return prob;
  };

  if (warp >= kWsConsumers) {
    // ----------------------------------------------------------------- producers ----
    asm volatile("setmaxnreg.dec.sync.aligned.u32 48;");
    const int pw = warp - kWsConsumers;
    if (solo && pw != 0) return;
    uint32_t issued = 0, c_phase = 0;
    bool ok = true, c_in_flight = false;
    SkWalk<SK> walk;
    walk.init(sk, num_tiles, num_kb);
    uint32_t tile, kb0, kb1;
    while (ok && walk.next(&tile, &kb0, &kb1)) {
      uint32_t tile_m, tile_n;
      const uint32_t prob = locate(tile, &tile_m, &tile_n);
      const uint32_t m0 = tile_m * BM, n0 = tile_n * kWsBN;
      const bool a_inside = m0 + BM <= p.m, b_inside = n0 + kWsBN <= p.n;
      // Only the CTA that holds a tile's first slabs applies alpha / beta and touches C (always, when the
      // contraction is not split).  The epilogue's C lines are requested from L2 24 slabs before the
      // item's last one; the staged C a few slabs into the item: by then the consumers are past the
      // previous tile's epilogue, so the wait for the buffer does not hold up the slab ring.
      const bool epilogue_here = kb0 == 0u;
      const uint32_t len = kb1 - kb0;
      const uint32_t c_prefetch_kb = len > 24u ? kb1 - 24u : kb0;
      const uint32_t c_stage_kb = kb0 + (len > 4u ? 4u : len - 1u);
      for (uint32_t kb = kb0; kb < kb1; ++kb) {
        if (stage_c && epilogue_here && pw == 0 && kb == c_stage_kb) {
          if (!mbar_wait(smem_u32(&c_empty_bar), c_phase ^ 1u, &abort_flag, kFaultWaitCLoad, 0)) {
            ok = false;
            break;
          }
          if (lane == 0) {
            mbar_expect_tx(smem_u32(&c_full_bar), T::kCDoubles * 8u);
            tma_load_tile(batched, smem_u32(c_smem), &tmap_c, smem_u32(&c_full_bar), (int32_t)m0, (int32_t)n0, (int32_t)prob);
          }
          c_in_flight = true;
          c_phase ^= 1u;
        }
        if (p.beta != 0.0 && !stage_c && epilogue_here && kb == c_prefetch_kb) {
          // Ask L2 for this tile's C: a bulk prefetch (the 1-D form of the TMA prefetch) per column
          // where the column pieces are 16-byte aligned, else one prefetch per 128-byte line.
          const uint32_t rows = p.m - m0 < (uint32_t)BM ? p.m - m0 : (uint32_t)BM;
          const double* __restrict__ Cp = C + (size_t)prob * p.batch_c;
          const bool c_bulk = ((reinterpret_cast<uintptr_t>(Cp) & 15u) == 0) && (p.ldc & 1u) == 0 && (rows & 1u) == 0;
          const uint32_t c_first = solo ? 0u : 16u * pw, c_last = solo ? (uint32_t)kWsBN : 16u * pw + 16u;
          if (c_bulk) {
            for (uint32_t c = c_first + lane; c < c_last; c += 32) {
              const uint32_t col = n0 + c;
              if (col < p.n)
                asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(Cp + (size_t)col * p.ldc + m0), "r"(rows * 8u)
                             : "memory");
            }
          } else {
            for (uint32_t c = c_first; c < c_last; c += 16) {
              const uint32_t col = n0 + c + (lane >> 1);
              if (col < p.n) {
                const double* c_col = Cp + (size_t)col * p.ldc + m0;
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
        const uint32_t slab_a = smem_a + stage * SA::kBytes, slab_b = smem_b + stage * SB::kBytes;
        if (pw == 0 && lane == 0) {
          // a box is always delivered whole (what lies outside the matrix arrives as zeros)
          const uint32_t tx = (p.tma_a ? SA::kBytes : 0u) + (p.tma_b ? SB::kBytes : 0u);
          if (tx) mbar_expect_tx(full, tx);
          else mbar_arrive(full);
          // coordinates: (contiguous index, other index)
          if (p.tma_a) tma_load_tile(batched, slab_a, &tmap_a, full, A_KMAJOR ? (int32_t)l0 : (int32_t)m0, A_KMAJOR ? (int32_t)m0 : (int32_t)l0, (int32_t)prob);
          if (p.tma_b) tma_load_tile(batched, slab_b, &tmap_b, full, B_KMAJOR ? (int32_t)l0 : (int32_t)n0, B_KMAJOR ? (int32_t)n0 : (int32_t)l0, (int32_t)prob);
        }
        if (!p.tma_a) {
          const double* __restrict__ Ap = A + (size_t)prob * p.batch_a;
          if (whole && a_inside) ws_fill_elements<BM, A_KMAJOR, false, kWsProducers>(slab_a, Ap, p.lda, m0, l0, p.m, p.k, lane, pw);
          else ws_fill_elements<BM, A_KMAJOR, true, kWsProducers>(slab_a, Ap, p.lda, m0, l0, p.m, p.k, lane, pw);
        }
        if (!p.tma_b) {
          const double* __restrict__ Bp = B + (size_t)prob * p.batch_b;
          if (whole && b_inside) ws_fill_elements<kWsBN, B_KMAJOR, false, kWsProducers>(slab_b, Bp, p.ldb, n0, l0, p.n, p.k, lane, pw);
          else ws_fill_elements<kWsBN, B_KMAJOR, true, kWsProducers>(slab_b, Bp, p.ldb, n0, l0, p.n, p.k, lane, pw);
        }
        ws_cp_async_arrive(full);
        ++issued;
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
      }
    }
    if (!ok || abort_flag) {
      // Leave only after the copies in flight have landed: the element copies of this warp, and
      // the TMA boxes of the slabs issued last (a short bounded wait on their full barriers).
      ws_cp_async_wait_all();
      if (c_in_flight && pw == 0) {  // the last staged C may still be landing
        const uint64_t t0 = global_timer_ns();
        while (!mbar_try_wait(smem_u32(&c_full_bar), c_phase ^ 1u) && global_timer_ns() - t0 < MMBO_DRAIN_LIMIT_NS) {
        }
      }
      const uint32_t pending = issued < (uint32_t)kStages ? issued : (uint32_t)kStages;
      for (uint32_t i = 0; pw == 0 && i < pending; ++i) {
        stage = stage == 0 ? kStages - 1 : stage - 1;
        if (stage == (uint32_t)kStages - 1) phase ^= 1u;
        const uint64_t t0 = global_timer_ns();
        while (!mbar_try_wait(smem_u32(&full_bar[stage]), phase) && global_timer_ns() - t0 < MMBO_DRAIN_LIMIT_NS) {
        }
      }
    }
    return;
  }

  // -------------------------------------------------------------------- consumers ----
  asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
  const int gid = lane >> 2, tig = lane & 3;                    // fragment coordinates of m8n8k4
  const int wm = (warp & 1) * (BM / 2), wn = (warp >> 1) * 32;  // this warp's (BM / 2) x 32 piece of the tile
  const double alpha = p.alpha, beta = p.beta;
  uint32_t c_phase = 0;
  SkWalk<SK> walk;
  walk.init(sk, num_tiles, num_kb);
  uint32_t tile, kb0, kb1;
  constexpr uint32_t kAccPerThread = kFragM * 8;  // accumulator doubles of one consumer thread
  while (walk.next(&tile, &kb0, &kb1)) {
    uint32_t tile_m, tile_n;
    const uint32_t prob = locate(tile, &tile_m, &tile_n);
    double* __restrict__ Cp = C + (size_t)prob * p.batch_c;
    const uint32_t m0 = tile_m * BM, n0 = tile_n * kWsBN;
    double acc[kFragM][4][2];
#pragma unroll
    for (int i = 0; i < kFragM; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;

    for (uint32_t kb = kb0; kb < kb1; ++kb) {
      if (!mbar_wait(smem_u32(&full_bar[stage]), phase, &abort_flag, kFaultWaitFull, stage)) return;
      // element (row, k) of a slab: SA::at / SB::at; this lane's fragments start at (w + gid, tig)
      const double* __restrict__ a_s = ws_smem + stage * SA::kDoubles + SA::at(wm + gid, tig);
      const double* __restrict__ b_s = ws_smem + kStages * SA::kDoubles + stage * SB::kDoubles + SB::at(wn + gid, tig);
#pragma unroll
      for (int k4 = 0; k4 < kWsBK; k4 += 4) {
        double fa[kFragM], fb[4];
#pragma unroll
        for (int i = 0; i < kFragM; ++i) fa[i] = a_s[SA::at(8 * i, k4)];  // A[m = gid][k = tig]
#pragma unroll
        for (int j = 0; j < 4; ++j) fb[j] = b_s[SB::at(8 * j, k4)];       // B[k = tig][n = gid]
#pragma unroll
        for (int i = 0; i < kFragM; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) dmma_m8n8k4(acc[i][j], fa[i], fb[j]);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&empty_bar[stage]));
      if (++stage == kStages) { stage = 0; phase ^= 1u; }
    }

    if (SK && kb0 != 0u) {
      // A later piece of a tile whose first slabs another CTA holds: hand the partial sums over
      // (value v of thread t at [(cta * N + v) * 128 + t]; the owner's thread t reads them back),
      // then raise this warp's flag.
      double* part = static_cast<double*>(sk.partials) + (size_t)blockIdx.x * kAccPerThread * 128u + tid;
#pragma unroll
      for (int i = 0; i < kFragM; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          __stcg(part + (size_t)((i * 4 + j) * 2 + 0) * 128u, acc[i][j][0]);
          __stcg(part + (size_t)((i * 4 + j) * 2 + 1) * 128u, acc[i][j][1]);
        }
      __threadfence();
      __syncwarp();
      if (lane == 0) sk_store_flag(sk.flags + blockIdx.x * kWsConsumers + warp, sk.epoch);
      continue;
    }
    if (SK && kb1 != num_kb) {
      // First slabs of a tile that continues in the next CTAs' runs (each reaches its piece first
      // thing): add their partial sums in CTA order, then finish the tile here.
      const unsigned long long units = (unsigned long long)num_tiles * num_kb;
      uint32_t have = kb1, j = blockIdx.x + 1u;
      while (have < num_kb && j < gridDim.x) {
        const unsigned long long run = sk_first_unit(units, j + 1u, gridDim.x) - sk_first_unit(units, j, gridDim.x);
        const uint32_t piece = run < (unsigned long long)(num_kb - have) ? (uint32_t)run : num_kb - have;
        if (piece != 0u) {
          if (!sk_wait_flag(sk.flags + j * kWsConsumers + warp, sk.epoch, &abort_flag, j)) return;
          const double* part = static_cast<const double*>(sk.partials) + (size_t)j * kAccPerThread * 128u + tid;
#pragma unroll
          for (int i = 0; i < kFragM; ++i)
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
              acc[i][jj][0] += __ldcg(part + (size_t)((i * 4 + jj) * 2 + 0) * 128u);
              acc[i][jj][1] += __ldcg(part + (size_t)((i * 4 + jj) * 2 + 1) * 128u);
            }
        }
        have += piece;
        ++j;
      }
    }

    // accumulator (i, j): C[m = gid][n = 2*tig + {0, 1}] of the 8 x 8 block at (wm + 8i, wn + 8j).
    // C is read 32 values per thread at a time (four columns x eight row blocks, all loads of a
    // round before their first use) and the tile is done in two such rounds.
    if (stage_c) {
      // old C from shared memory (element (row, col) of the tile at c_smem[col * kCPitch + row])
      if (!mbar_wait(smem_u32(&c_full_bar), c_phase, &abort_flag, kFaultWaitCLoad, 1)) return;
      c_phase ^= 1u;
      const uint32_t row = m0 + wm + gid;
      const uint32_t rows_left = p.m > row ? p.m - row : 0u;
      const double* __restrict__ c_s = c_smem + wm + gid;
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const uint32_t cl = wn + 8 * j + 2 * tig + e, col = n0 + cl;
          double* __restrict__ c_col = Cp + (size_t)col * p.ldc + row;
#pragma unroll
          for (int i = 0; i < kFragM; ++i) {
            const double old = c_s[cl * T::kCPitch + 8 * i];
            if (col < p.n && 8u * i < rows_left && (p.diag & 1u) == 0u) c_col[8 * i] = fma(beta, old, alpha * acc[i][j][e]);
          }
        }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&c_empty_bar));  // this warp has read its part of the staged tile
    } else if ((p.diag & 1u) == 0u) {
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
          c_col[q] = Cp + (size_t)col * p.ldc + row;
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
