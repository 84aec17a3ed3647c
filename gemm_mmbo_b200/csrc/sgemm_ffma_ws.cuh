// SGEMM on the CUDA cores (exact fp32 products and sums), warp-specialised and persistent:
// the arrangement of the fp64 tensor kernel (dgemm_dmma_ws.cuh) with an FFMA micro-kernel.
//   * a producer warpgroup (four warps, 32 registers each after setmaxnreg) fills a ring of
//     128 x 16 operand slabs [k][128 + 4].  An operand whose tile rows are contiguous in memory
//     (A not transposed, B transposed) with a 16-byte aligned base and a leading dimension that is
//     a multiple of 4 comes in through TMA, one box per slab, four elements wider than the tile
//     so that the copy engine itself produces the padded pitch; edges and the K tail arrive as
//     zeros.  Any other operand (K-contiguous, odd leading dimension, unaligned base) is
//     filled by the 128 producer lanes with 4-byte cp.async copies that transpose where needed
//     and zero-fill outside the matrix;
//   * two consumer warpgroups (eight warps, 104 registers each): 16 x 16 threads, 8 x 8
//     accumulators per thread held as packed pairs and updated with fma.rn.f32x2, fragments
//     read with 128-bit loads; no block barrier in the main loop (full / empty mbarriers);
//   * two CTAs per SM, tiles of the remapped order walked with a stride of the grid.
// Every wait is bounded (ptx.cuh).  The write rule is the reference's
// (src/gemm/ref/Kernels.cpp:87); counterpart of its register-tiled kernels
// (e.g. MT128x128x08 in src/gemm/constants.h:20-33).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "dgemm_dmma_ws.cuh"  // ws_cp_async_arrive, ws_cp_async_wait_all
#include "ptx.cuh"
#include "raster.h"
#include "sgemm_ffma.cuh"  // SgemmParams
#include "stream_k.cuh"

namespace mmbo {

constexpr int kFwBM = 128, kFwBN = 128, kFwBK = 16, kFwStages = 4, kFwPad = 4;
constexpr int kFwPitch = kFwBM + kFwPad;             // floats; same for both operands (BM == BN)
constexpr int kFwSlabFloats = kFwBK * kFwPitch;      // one operand slab
constexpr uint32_t kFwSlabBytes = kFwSlabFloats * 4u;
constexpr int kFwConsumerWarps = 8, kFwProducerWarps = 4;
constexpr int kFwThreads = (kFwConsumerWarps + kFwProducerWarps) * 32;
constexpr size_t kFwSmemBytes = (size_t)kFwStages * 2 * kFwSlabBytes + 128;
constexpr uint32_t kFwFullCount = kFwProducerWarps * 32 + 1;

struct SgemmWsFlags {
  uint32_t tma_a, tma_b;  // the operand is addressed through its tensor map
};

__device__ __forceinline__ void fw_cp_async_4(uint32_t smem_dst, const void* gmem_src, bool valid) {
  const uint32_t bytes = valid ? 4u : 0u;  // source size 0: the slot is zero-filled
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_dst), "l"(gmem_src), "r"(bytes) : "memory");
}

// Element-wise slab fill by the 128 producer lanes (always guarded).  CONTIG_ROW: the tile-row
// index is the contiguous one in memory; otherwise k is and the copy transposes.
template <bool CONTIG_ROW>
__device__ __forceinline__ void fw_fill_elements(uint32_t slab, const float* __restrict__ base, uint32_t ld,
                                                 uint32_t row0, uint32_t l0, uint32_t row_end, uint32_t l_end,
                                                 int pt) {  // pt = 0..127, index among the producer lanes
  if constexpr (CONTIG_ROW) {  // lane pt copies row pt of every k-row
    const bool row_ok = row0 + pt < row_end;
    const float* src = base + (size_t)row0 + pt + (size_t)l0 * ld;
#pragma unroll 4
    for (int l = 0; l < kFwBK; ++l) {
      const bool ok = row_ok && l0 + l < l_end;
      fw_cp_async_4(slab + (l * kFwPitch + pt) * 4u, ok ? src : base, ok);
      src += ld;
    }
  } else {  // 16 consecutive k of 8 rows per pass of the 128 lanes
    const uint32_t l = pt & 15, r = pt >> 4;
    const bool l_ok = l0 + l < l_end;
    const float* src = base + (size_t)(l0 + l) + (size_t)(row0 + r) * ld;
    const size_t step = 8 * (size_t)ld;
#pragma unroll 4
    for (int e = 0; e < kFwBM / 8; ++e) {
      const bool ok = l_ok && row0 + r + 8 * e < row_end;
      fw_cp_async_4(slab + (l * kFwPitch + r + 8 * e) * 4u, ok ? src : base, ok);
      src += step;
    }
  }
}

template <bool TRANS_A, bool TRANS_B, bool SK = false>
__global__ void __launch_bounds__(kFwThreads, 2)
sgemm_ffma_ws_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                     const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C,
                     const SgemmParams p, const SgemmWsFlags f, const StreamK sk) {
  extern __shared__ __align__(16) uint8_t fw_smem_raw[];
  float* const smem = reinterpret_cast<float*>(fw_smem_raw + ((128u - (smem_u32(fw_smem_raw) & 127u)) & 127u));
  __shared__ __align__(8) uint64_t full_bar[kFwStages], empty_bar[kFwStages];
  __shared__ uint32_t abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t smem_a = smem_u32(smem), smem_b = smem_a + kFwStages * kFwSlabBytes;
  const bool solo = f.tma_a && f.tma_b;  // one producer warp feeds alone, the others leave
  if (tid == 0) {
    abort_flag = 0;
    for (int s = 0; s < kFwStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), solo ? 33u : kFwFullCount);
      mbar_init(smem_u32(&empty_bar[s]), kFwConsumerWarps);
    }
    fence_mbar_init();
  }
  __syncthreads();

  const uint32_t tiles_m = (p.m + kFwBM - 1) / kFwBM, tiles_n = (p.n + kFwBN - 1) / kFwBN;
  const uint32_t num_tiles = tiles_m * tiles_n;
  const uint32_t num_kb = (p.k + kFwBK - 1) / kFwBK;
  uint32_t stage = 0, phase = 0;

  if (warp >= kFwConsumerWarps) {
    // ----------------------------------------------------------------- producers ----
    asm volatile("setmaxnreg.dec.sync.aligned.u32 32;");
    const int pw = warp - kFwConsumerWarps, pt = pw * 32 + lane;
    if (solo && pw != 0) return;
    uint32_t issued = 0;
    bool ok = true;
    SkWalk<SK> walk;
    walk.init(sk, num_tiles, num_kb);
    uint32_t tile, kb0, kb1;
    while (ok && walk.next(&tile, &kb0, &kb1)) {
      uint32_t tile_m, tile_n;
      mmbo_tile_from_serial(tile, tiles_m, tiles_n, p.wgm, &tile_m, &tile_n);
      const uint32_t m0 = tile_m * kFwBM, n0 = tile_n * kFwBN;
      for (uint32_t kb = kb0; kb < kb1; ++kb) {
        const uint32_t full = smem_u32(&full_bar[stage]);
        if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, &abort_flag, kFaultWaitEmpty, stage)) {
          ok = false;
          break;
        }
        const uint32_t l0 = kb * kFwBK;
        const uint32_t slab_a = smem_a + stage * kFwSlabBytes, slab_b = smem_b + stage * kFwSlabBytes;
        if (pw == 0 && lane == 0) {
          const uint32_t tx = (f.tma_a ? kFwSlabBytes : 0u) + (f.tma_b ? kFwSlabBytes : 0u);
          if (tx) mbar_expect_tx(full, tx);
          else mbar_arrive(full);
          if (f.tma_a) tma_load_2d(slab_a, &tmap_a, full, (int32_t)m0, (int32_t)l0);
          if (f.tma_b) tma_load_2d(slab_b, &tmap_b, full, (int32_t)n0, (int32_t)l0);
        }
        if (!f.tma_a) fw_fill_elements<!TRANS_A>(slab_a, A, p.lda, m0, l0, p.m, p.k, pt);
        if (!f.tma_b) fw_fill_elements<TRANS_B>(slab_b, B, p.ldb, n0, l0, p.n, p.k, pt);
        ws_cp_async_arrive(full);
        ++issued;
        if (++stage == kFwStages) { stage = 0; phase ^= 1u; }
      }
    }
    if (!ok || abort_flag) {
      ws_cp_async_wait_all();
      const uint32_t pending = issued < (uint32_t)kFwStages ? issued : (uint32_t)kFwStages;
      for (uint32_t i = 0; pw == 0 && i < pending; ++i) {
        stage = stage == 0 ? kFwStages - 1 : stage - 1;
        if (stage == (uint32_t)kFwStages - 1) phase ^= 1u;
        const uint64_t t0 = global_timer_ns();
        while (!mbar_try_wait(smem_u32(&full_bar[stage]), phase) && global_timer_ns() - t0 < MMBO_DRAIN_LIMIT_NS) {
        }
      }
    }
    return;
  }

  // -------------------------------------------------------------------- consumers ----
  asm volatile("setmaxnreg.inc.sync.aligned.u32 104;");
  const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads; m = h * 64 + tx * 4 + e, n = h * 64 + ty * 4 + e
  const float alpha = p.alpha, beta = p.beta;
  const bool use_c = beta != 0.f;
  SkWalk<SK> walk;
  walk.init(sk, num_tiles, num_kb);
  uint32_t tile, kb0, kb1;
  constexpr uint32_t kConsumerThreads = kFwConsumerWarps * 32;
  while (walk.next(&tile, &kb0, &kb1)) {
    uint32_t tile_m, tile_n;
    mmbo_tile_from_serial(tile, tiles_m, tiles_n, p.wgm, &tile_m, &tile_n);
    const uint32_t m0 = tile_m * kFwBM, n0 = tile_n * kFwBN;
    uint64_t acc2[8][4];  // [n index][pair of m indices]
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc2[j][i] = 0ull;

    for (uint32_t kb = kb0; kb < kb1; ++kb) {
      if (!mbar_wait(smem_u32(&full_bar[stage]), phase, &abort_flag, kFaultWaitFull, stage)) return;
      const float* __restrict__ a_s = smem + stage * kFwSlabFloats + tx * 4;
      const float* __restrict__ b_s = smem + (kFwStages + stage) * kFwSlabFloats + ty * 4;
#pragma unroll
      for (int l = 0; l < kFwBK; ++l) {
        uint64_t fa2[4];
        float fb[8];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint4 x = *reinterpret_cast<const uint4*>(a_s + l * kFwPitch + h * 64);
          fa2[2 * h] = pack_f32x2(x.x, x.y);
          fa2[2 * h + 1] = pack_f32x2(x.z, x.w);
          const float4 y = *reinterpret_cast<const float4*>(b_s + l * kFwPitch + h * 64);
          fb[4 * h] = y.x; fb[4 * h + 1] = y.y; fb[4 * h + 2] = y.z; fb[4 * h + 3] = y.w;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint64_t bb = pack_f32x2(__float_as_uint(fb[j]), __float_as_uint(fb[j]));
#pragma unroll
          for (int i = 0; i < 4; ++i) acc2[j][i] = fma_f32x2(fa2[i], bb, acc2[j][i]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&empty_bar[stage]));
      if (++stage == kFwStages) { stage = 0; phase ^= 1u; }
    }

    if (SK && kb0 != 0u) {
      // A later piece of a tile whose first slabs another CTA holds: hand the partial sums over (pair v of
      // thread t at [(cta * 32 + v) * 256 + t]) and raise this warp's flag.
      unsigned long long* part = static_cast<unsigned long long*>(sk.partials) + (size_t)blockIdx.x * 32u * kConsumerThreads + tid;
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) __stcg(part + (size_t)(j * 4 + i) * kConsumerThreads, (unsigned long long)acc2[j][i]);
      __threadfence();
      __syncwarp();
      if (lane == 0) sk_store_flag(sk.flags + blockIdx.x * kFwConsumerWarps + warp, sk.epoch);
      continue;
    }
    if (SK && kb1 != num_kb) {
      // First slabs of a tile that continues in the next CTAs' runs: add their partial sums in CTA order.
      const unsigned long long units = (unsigned long long)num_tiles * num_kb;
      const uint64_t one2 = pack_f32x2(0x3f800000u, 0x3f800000u);
      uint32_t have = kb1, jc = blockIdx.x + 1u;
      while (have < num_kb && jc < gridDim.x) {
        const unsigned long long run = sk_first_unit(units, jc + 1u, gridDim.x) - sk_first_unit(units, jc, gridDim.x);
        const uint32_t piece = run < (unsigned long long)(num_kb - have) ? (uint32_t)run : num_kb - have;
        if (piece != 0u) {
          if (!sk_wait_flag(sk.flags + jc * kFwConsumerWarps + warp, sk.epoch, &abort_flag, jc)) return;
          const unsigned long long* part =
              static_cast<const unsigned long long*>(sk.partials) + (size_t)jc * 32u * kConsumerThreads + tid;
#pragma unroll
          for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i)  // acc + 1 * partial, each half rounded as a scalar add
              acc2[j][i] = fma_f32x2(one2, (uint64_t)__ldcg(part + (size_t)(j * 4 + i) * kConsumerThreads), acc2[j][i]);
        }
        have += piece;
        ++jc;
      }
    }

    // Write-back: C = beta != 0 ? alpha*acc + beta*C : alpha*acc.
#pragma unroll
    for (int hn = 0; hn < 2; ++hn)
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const uint32_t j = n0 + hn * 64 + ty * 4 + jj;
        if (j >= p.n) continue;
#pragma unroll
        for (int hm = 0; hm < 2; ++hm) {
          const uint32_t i = m0 + hm * 64 + tx * 4;
          if (i >= p.m) continue;
          float* cp = C + (size_t)i + (size_t)j * p.ldc;
          float a4[4];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const uint64_t v = acc2[hn * 4 + jj][hm * 2 + e];
            a4[2 * e] = __uint_as_float((uint32_t)(v & 0xffffffffull));
            a4[2 * e + 1] = __uint_as_float((uint32_t)(v >> 32));
          }
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
}

}  // namespace mmbo
