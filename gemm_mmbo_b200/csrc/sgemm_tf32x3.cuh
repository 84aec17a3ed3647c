// SGEMM on the sm_100a tensor cores with fp32-level accuracy ("3xTF32"):
//   C = alpha * op(A) * op(B) + beta * C,  fp32 storage.
//
// Every fp32 operand element x is split into x = hi + lo with hi = tf32(x) and
// lo = tf32(x - hi); the product is accumulated as  lo*hi + hi*lo + hi*hi  by three
// tcgen05.mma.kind::tf32 instructions per K step into one fp32 accumulator in tensor
// memory.  The dropped lo*lo term and the rounding of lo are of relative size 2^-22,
// which keeps the result inside the fp32 tolerance of the benchmark (relative
// Frobenius error 1e-5) while running on the tensor pipe instead of the FFMA pipe.
//
// Tensor-core fp32 accumulation truncates: a chain of a few thousand dependent
// accumulations drifts by several 1e-5 relative, which is outside the fp32 tolerance.
// The kernel therefore keeps every accumulation chain in tensor memory short (`chunk`
// stages of 32 values of k, 4 by default: measured relative Frobenius error at k = 8192
// is 0.9e-6 with 4, 1.8e-6 with 8, 7.2e-6 with 32, 5.7e-5 with one chain), and the epilogue warps add the finished partial sums into
// fp32 registers with round-to-nearest FADDs while the UMMA issuer already fills the
// other accumulator buffer.
//
// Two kernels:
//   split_pack_kernel   reads op(A) (or op(B)^T) in whatever layout and leading
//                       dimension the caller has, and writes hi and lo parts into
//                       scratch memory as K-major rows of Kpad floats (Kpad a multiple
//                       of 32, so that rows are 128-byte multiples and TMA can address
//                       them whatever the caller's alignment);
//   sgemm_tf32x3_kernel the tcgen05 GEMM over the packed operands: same roles, ring
//                       of TMA stages, double-buffered tensor-memory accumulators,
//                       CTA pairs and persistent tile walk as hgemm_tcgen05_kernel.
// The epilogue goes through TMA when C allows it (16-byte aligned base, ldc % 4 == 0)
// and through coalesced plain loads/stores otherwise, so padded leading dimensions
// such as ld = dim + 3 stay on this path.
//
// Counterpart in the reference: the general kernel body src/gemm/ref/Kernels.cpp:153-1123
// (same write rule :87; beta == 0 never reads C).
#pragma once

#include "ptx.cuh"
#include "raster.h"

namespace mmbo {

__device__ __forceinline__ float round_tf32(float x) {
  uint32_t u;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
  return __uint_as_float(u);
}

// X holds a logical R x K operand: element (r, l) at X[r + l*ld] when ROW_CONTIG, at
// X[l + r*ld] otherwise.  hi/lo: R rows of Kpad floats, element (r, l) at [r*Kpad + l],
// Kpad a multiple of 32 and the arrays 16-byte aligned (they are this library's scratch),
// so every store is a 16-byte store whatever the caller's layout.  Columns l >= K of
// the scratch rows may receive zeros; the GEMM never reads them (its tensor maps end at
// K).  One block handles a 64 x 64 tile: 16 coalesced 4-byte loads in flight per thread.
constexpr int kSplitTile = 64;
template <bool ROW_CONTIG>
__global__ void __launch_bounds__(256)
split_pack_kernel(const float* __restrict__ X, size_t ld, uint32_t R, uint32_t K, uint32_t Kpad,
                  float* __restrict__ hi, float* __restrict__ lo, size_t x_batch_stride) {
  __shared__ float tile[kSplitTile][kSplitTile + 1];  // [l][r], used by the transposing variant
  const uint32_t tid = threadIdx.x;
  // strided batch: problem blockIdx.z; its packed rows follow the previous problem's
  X += (size_t)blockIdx.z * x_batch_stride;
  hi += (size_t)blockIdx.z * R * Kpad;
  lo += (size_t)blockIdx.z * R * Kpad;
  const uint32_t l0 = blockIdx.x * kSplitTile, r0 = blockIdx.y * kSplitTile;
  if (ROW_CONTIG) {
#pragma unroll
    for (uint32_t i = 0; i < 16; ++i) {
      const uint32_t idx = tid + 256u * i, r = idx % kSplitTile, l = idx / kSplitTile;
      tile[l][r] = (l0 + l < K && r0 + r < R) ? X[(size_t)(r0 + r) + (size_t)(l0 + l) * ld] : 0.f;
    }
    __syncthreads();
  }
#pragma unroll
  for (uint32_t j = 0; j < 4; ++j) {
    const uint32_t idx = tid + 256u * j, l4 = (idx % 16u) * 4u, r = idx / 16u;
    if (r0 + r >= R || l0 + l4 >= Kpad) continue;
    float x[4];
#pragma unroll
    for (uint32_t e = 0; e < 4; ++e) {
      if (ROW_CONTIG) x[e] = tile[l4 + e][r];
      else x[e] = (l0 + l4 + e < K) ? X[(size_t)(l0 + l4 + e) + (size_t)(r0 + r) * ld] : 0.f;
    }
    float4 h, d;
    h.x = round_tf32(x[0]); h.y = round_tf32(x[1]); h.z = round_tf32(x[2]); h.w = round_tf32(x[3]);
    d.x = round_tf32(x[0] - h.x); d.y = round_tf32(x[1] - h.y);
    d.z = round_tf32(x[2] - h.z); d.w = round_tf32(x[3] - h.w);
    const size_t off = (size_t)(r0 + r) * Kpad + l0 + l4;
    *reinterpret_cast<float4*>(hi + off) = h;
    *reinterpret_cast<float4*>(lo + off) = d;
  }
}

constexpr int kTfTileN = 128;  // problem-N extent per CTA = UMMA M per CTA
constexpr int kTfBlockK = 32;  // floats per stage along K = one 128-byte swizzle row
constexpr int kTfUmmaK = 8;    // K extent of one kind::tf32 UMMA
constexpr int kTfEpiBufBytes = 32 * 128;  // 32 C columns x 32 rows of fp32
constexpr int kTfSums = 128;   // running sums (accumulator columns) one epilogue thread keeps in registers

// EW epilogue warps: 4 (tile of 128 rows of C: every warp owns all 128 accumulator columns
// of its lane quarter) or 8 (tile of 256 rows: two warps per quarter, 128 columns each).
// With 8 the block has three warpgroups -- {producer, issuer, 2 idle warps}, {4 epilogue
// warps}, {4 epilogue warps} -- so that the first can hand registers to the other two.
template <int TM, int STAGES, int CG, int EW = 4>
struct TfSmem {
  static constexpr int kThreads = EW == 4 ? 192 : 384;
  static constexpr int kFirstEpiWarp = EW == 4 ? 2 : 4;
  static constexpr int kBufsPerWarp = EW == 4 ? 2 : 1;
  static constexpr int kAopRows = TM / CG;
  static constexpr int kBopBytes = kTfTileN * 128;  // one of hi / lo
  static constexpr int kAopBytes = kAopRows * 128;
  static constexpr int kStageBytes = 2 * (kBopBytes + kAopBytes);  // Bhi, Blo, Ahi, Alo
  static constexpr int kEpiOffset = STAGES * kStageBytes;
  static constexpr int kEpiBytes = EW * kBufsPerWarp * kTfEpiBufBytes;
  static constexpr int kBarOffset = kEpiOffset + kEpiBytes;
  static constexpr int kNumBars = 2 * STAGES + 4 + 2 * EW;
  static constexpr int kMiscOffset = kBarOffset + kNumBars * 8;
  static constexpr int kTotal = kMiscOffset + 16;
  static constexpr int kDynamic = kTotal + 1024;
};

struct TfParams {
  uint32_t m, n, k;
  uint32_t tiles_m, tiles_n;
  uint32_t batch;                     // problems of a strided batch; the walk covers batch * tiles_m * tiles_n tiles
  unsigned long long c_batch_stride;  // elements between the C of consecutive problems (plain epilogue)
  uint32_t wgm;
  MmboTileWalk walk;  // the walk with its divisions precomputed (mmbo_tile_walk_make(tiles_m, tiles_n, wgm))
  float alpha, beta;
  float* c;        // used by the plain epilogue
  uint32_t ldc;
  uint32_t c_tma;  // 1: C is read/written through the tensor map
  uint32_t chunk;  // stages accumulated in tensor memory before the partial sum is drained
};

template <int TM, int STAGES, int CG, int EW = 4>
__global__ void __launch_bounds__(EW == 4 ? 192 : 384, 1)
sgemm_tf32x3_kernel(const __grid_constant__ CUtensorMap tmap_a_hi, const __grid_constant__ CUtensorMap tmap_a_lo,
                    const __grid_constant__ CUtensorMap tmap_b_hi, const __grid_constant__ CUtensorMap tmap_b_lo,
                    const __grid_constant__ CUtensorMap tmap_c, const TfParams p) {
  using L = TfSmem<TM, STAGES, CG, EW>;
  static_assert(TM == kTfSums * (EW / 4), "one epilogue thread keeps 128 running sums in registers");
  constexpr uint32_t kTmemCols = 2 * TM;  // two partial-sum buffers

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + L::kBarOffset;
  auto full_bar = [&](uint32_t s) { return bar_base + 8u * s; };
  auto empty_bar = [&](uint32_t s) { return bar_base + 8u * (STAGES + s); };
  auto tmem_full_bar = [&](uint32_t a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tmem_empty_bar = [&](uint32_t a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  auto cload_bar = [&](uint32_t w, uint32_t b) { return bar_base + 8u * (2 * STAGES + 4 + 2 * w + b); };
  volatile uint32_t* tmem_ptr_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kMiscOffset);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kMiscOffset + 4);

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  uint32_t cta_rank = 0;
  if constexpr (CG == 2) asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(cta_rank));
  const uint32_t walker = blockIdx.x / CG, num_walkers = gridDim.x / CG;
  const uint32_t tiles_per_problem = p.tiles_m * p.tiles_n;
  const uint32_t num_tiles = tiles_per_problem * p.batch;
  const uint32_t num_kb = (p.k + kTfBlockK - 1) / kTfBlockK;
  const bool batched = p.batch > 1u;  // 3-D tensor maps; single problems keep the 2-D forms
  auto locate = [&](uint32_t tile, uint32_t* tm, uint32_t* tn) -> uint32_t {
    const uint32_t prob = batched ? mmbo_fastdiv(tile, p.walk.by_problem) : 0u;
    mmbo_tile_walk_locate(p.walk, tile - prob * tiles_per_problem, tm, tn);
    return prob;
  };

  if (threadIdx.x == 0) {
    *abort_flag = 0u;
    for (uint32_t s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (uint32_t a = 0; a < 2; ++a) {
      mbar_init(tmem_full_bar(a), 1);
      mbar_init(tmem_empty_bar(a), EW * CG);
    }
    for (uint32_t w = 0; w < EW; ++w)
      for (uint32_t b = 0; b < 2; ++b) mbar_init(cload_bar(w, b), 1);
    fence_mbar_init();
    prefetch_tensormap(&tmap_a_hi);
    prefetch_tensormap(&tmap_a_lo);
    prefetch_tensormap(&tmap_b_hi);
    prefetch_tensormap(&tmap_b_lo);
    if (p.c_tma) prefetch_tensormap(&tmap_c);
  }
  __syncwarp();
  if (warp == 1) {
    tmem_alloc<CG>(smem_u32(const_cast<uint32_t*>(tmem_ptr_slot)), kTmemCols);
    tmem_relinquish<CG>();
  }
  tcgen05_fence_before();
  __syncthreads();
  if constexpr (CG == 2) {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  }
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_ptr_slot;
  // Programmatic dependent launch: set-up done, nothing of global memory touched yet (the split pass that writes
  // this kernel's operands is the kernel before it in the stream).
  griddep_launch_dependents();
  griddep_wait();

  // With 8 epilogue warps (384 threads, 168 registers each at launch) the first warpgroup
  // hands registers to the two epilogue warpgroups, whose threads keep 128 running sums:
  // 56 / 224 / 224.  Each role branch opens with its own setmaxnreg so that the
  // assembler allocates registers per branch.
  if (warp == 0) {
    if constexpr (EW == 8) asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    // ===== TMA producer =====
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, issued = 0;
      bool ok = true;
      for (uint32_t tile = walker; ok && tile < num_tiles; tile += num_walkers) {
        uint32_t tm_idx, tn_idx;
        const int32_t prob = static_cast<int32_t>(locate(tile, &tm_idx, &tn_idx));
        const int32_t m0 = static_cast<int32_t>(tm_idx * TM + cta_rank * L::kAopRows);
        const int32_t n0 = static_cast<int32_t>((tn_idx * CG + cta_rank) * kTfTileN);
        for (uint32_t kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, kFaultWaitEmpty, stage)) {
            ok = false;
            break;
          }
          const uint32_t bar = (CG == 2) ? mapa_shared(full_bar(stage), 0u) : full_bar(stage);
          const uint32_t s0 = smem_base + stage * L::kStageBytes;
          const int32_t k0 = static_cast<int32_t>(kb * kTfBlockK);
          if (cta_rank == 0) mbar_expect_tx(full_bar(stage), L::kStageBytes * CG);
          auto load = [&](uint32_t dst, const CUtensorMap* map, int32_t c1) {
            if constexpr (CG == 2) tma_load_tile_pair(batched, dst, map, bar, k0, c1, prob);
            else tma_load_tile(batched, dst, map, bar, k0, c1, prob);
          };
          load(s0, &tmap_b_hi, n0);                                       // box {32 k, 128 n}
          load(s0 + L::kBopBytes, &tmap_b_lo, n0);
          load(s0 + 2 * L::kBopBytes, &tmap_a_hi, m0);                    // box {32 k, TM/CG m}
          load(s0 + 2 * L::kBopBytes + L::kAopBytes, &tmap_a_lo, m0);
          ++issued;
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok && cta_rank == 0) {
        // Unwind: wait (bounded) for the copies already issued into this ring.
        uint32_t s = stage, ph = phase;
        const uint32_t back = issued < STAGES ? issued : STAGES;
        for (uint32_t i = 0; i < back; ++i) {
          if (s == 0) {
            s = STAGES;
            ph ^= 1u;
          }
          --s;
          uint32_t none = 0;
          mbar_wait(full_bar(s), ph, &none, kFaultWaitFull, 0x100u + s, MMBO_DRAIN_LIMIT_NS);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if constexpr (EW == 8) asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    // ===== UMMA issuer (leader CTA of a pair) =====
    if (lane == 0 && cta_rank == 0) {
      constexpr uint32_t idesc = make_idesc(2u, 0u, 0u, kTfTileN * CG, TM);
      uint32_t stage = 0, phase = 0, chunk_ctr = 0;
      bool ok = true;
      for (uint32_t tile = walker; ok && tile < num_tiles; tile += num_walkers) {
        uint32_t acc = 0;
        for (uint32_t kb = 0; kb < num_kb; ++kb) {
          const uint32_t in_chunk = kb % p.chunk;
          if (in_chunk == 0) {
            // a fresh, short accumulation chain in the buffer the epilogue has drained
            acc = chunk_ctr & 1u;
            if (!mbar_wait(tmem_empty_bar(acc), ((chunk_ctr >> 1) & 1u) ^ 1u, abort_flag, kFaultWaitTmemEmpty,
                           acc)) {
              ok = false;
              break;
            }
            tcgen05_fence_after();
          }
          const uint32_t d_tmem = tmem_base + acc * TM;
          if (!mbar_wait(full_bar(stage), phase, abort_flag, kFaultWaitFull, stage)) {
            ok = false;
            break;
          }
          tcgen05_fence_after();
          const uint32_t s0 = smem_base + stage * L::kStageBytes;
          const uint64_t b_hi = make_smem_desc_sw128(s0, 16u, 1024u);
          const uint64_t b_lo = make_smem_desc_sw128(s0 + L::kBopBytes, 16u, 1024u);
          const uint64_t a_hi = make_smem_desc_sw128(s0 + 2 * L::kBopBytes, 16u, 1024u);
          const uint64_t a_lo = make_smem_desc_sw128(s0 + 2 * L::kBopBytes + L::kAopBytes, 16u, 1024u);
#pragma unroll
          for (uint32_t j = 0; j < kTfBlockK / kTfUmmaK; ++j) {
            const uint64_t adv = (j * 32u) >> 4;  // 8 floats = 32 bytes per K step
            // small cross terms first, the hi*hi term last
            umma_ss<CG, true>(d_tmem, b_lo + adv, a_hi + adv, idesc, (in_chunk | j) != 0u ? 1u : 0u);
            umma_ss<CG, true>(d_tmem, b_hi + adv, a_lo + adv, idesc, 1u);
            umma_ss<CG, true>(d_tmem, b_hi + adv, a_hi + adv, idesc, 1u);
          }
          if constexpr (CG == 2) umma_commit_pair(empty_bar(stage), 3);
          else umma_commit(empty_bar(stage));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
          if (in_chunk == p.chunk - 1 || kb == num_kb - 1) {  // partial sum complete
            if constexpr (CG == 2) umma_commit_pair(tmem_full_bar(acc), 3);
            else umma_commit(tmem_full_bar(acc));
            ++chunk_ctr;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp < L::kFirstEpiWarp) {
    if constexpr (EW == 8) asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");  // idle warps of the first warpgroup
  } else {
    if constexpr (EW == 8) asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    // ===== epilogue: warp owns tensor-memory lanes [32q, 32q+32) = 32 columns of C and
    // 128 accumulator columns (= rows of C) of them =====
    const uint32_t q = warp & 3u, epi_w = warp - L::kFirstEpiWarp;
    const uint32_t col_base = (epi_w >> 2) * kTfSums;
    const uint32_t buf_base = smem_base + L::kEpiOffset + epi_w * L::kBufsPerWarp * kTfEpiBufBytes;
    uint8_t* buf_gen = smem_gen + L::kEpiOffset + epi_w * L::kBufsPerWarp * kTfEpiBufBytes;
    const bool use_c = (p.beta != 0.0f);
    const bool c_tma = p.c_tma != 0u;
    const float alpha = p.alpha, beta = p.beta;
    const uint32_t num_chunks = (num_kb + p.chunk - 1) / p.chunk;
    uint32_t chunk_ctr = 0, out_ctr = 0;
    uint32_t cphase[2] = {0u, 0u};
    bool ok = true;
    for (uint32_t tile = walker; ok && tile < num_tiles; tile += num_walkers) {
      uint32_t tm_idx, tn_idx;
      const int32_t prob = static_cast<int32_t>(locate(tile, &tm_idx, &tn_idx));
      float* const c_plain = p.c + static_cast<size_t>(prob) * p.c_batch_stride;
      const uint32_t m0 = tm_idx * TM + col_base;
      const uint32_t ncol0 = (tn_idx * CG + cta_rank) * kTfTileN + 32u * q;
      // running sums of this thread's C column over the tile's TM rows
      float sums[kTfSums];
#pragma unroll
      for (int i = 0; i < kTfSums; ++i) sums[i] = 0.f;
      for (uint32_t ch = 0; ok && ch < num_chunks; ++ch, ++chunk_ctr) {
        const uint32_t acc = chunk_ctr & 1u, acc_phase = (chunk_ctr >> 1) & 1u;
        ok = mbar_wait_warp(tmem_full_bar(acc), acc_phase, abort_flag, kFaultWaitTmemFull, acc);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t t_warp = tmem_base + ((32u * q) << 16) + acc * TM + col_base;
        // two register buffers: the load of columns c+1 is in flight during the adds of c
        uint32_t r0[32], r1[32];
        tmem_ld_32x32(t_warp, r0);
#pragma unroll
        for (uint32_t c = 0; c < kTfSums / 32; c += 2) {
          tmem_ld_wait();
          tmem_ld_32x32(t_warp + 32u * (c + 1), r1);
#pragma unroll
          for (int e = 0; e < 32; ++e) sums[32 * c + e] += __uint_as_float(r0[e]);
          tmem_ld_wait();
          if (c + 2 < kTfSums / 32) tmem_ld_32x32(t_warp + 32u * (c + 2), r0);
#pragma unroll
          for (int e = 0; e < 32; ++e) sums[32 * (c + 1) + e] += __uint_as_float(r1[e]);
        }
        // partial sum consumed: hand the buffer back to the UMMA issuer
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) {
          if constexpr (CG == 2) mbar_arrive_cluster(mapa_shared(tmem_empty_bar(acc), 0u));
          else mbar_arrive(tmem_empty_bar(acc));
        }
      }
      if (!ok) break;
#pragma unroll
      for (uint32_t c = 0; c < kTfSums / 32; ++c, ++out_ctr) {
        const uint32_t b = L::kBufsPerWarp == 2 ? (out_ctr & 1u) : 0u;
        const uint32_t sbuf = buf_base + b * kTfEpiBufBytes;
        float* gbuf = reinterpret_cast<float*>(buf_gen + b * kTfEpiBufBytes);
        const uint32_t mrow0 = m0 + 32u * c;
        const bool in_range = (mrow0 < p.m) && (ncol0 < p.n);  // warp-uniform
        const bool load_c = use_c && in_range;
        // staging tile: row t = C column ncol0 + t, 32 floats = rows mrow0 .. mrow0+31;
        // 16-byte piece j of a row lives at piece (j ^ (t & 7)) (the 128-byte TMA swizzle)
        if (c_tma) {
          if (lane == 0) {  // this buffer's previous store has read it
            if constexpr (L::kBufsPerWarp == 2) tma_store_wait_read<1>();
            else tma_store_wait_read<0>();
          }
          __syncwarp();
          if (load_c && lane == 0) {
            mbar_expect_tx(cload_bar(epi_w, b), kTfEpiBufBytes);
            tma_load_tile(batched, sbuf, &tmap_c, cload_bar(epi_w, b), static_cast<int32_t>(mrow0),
                        static_cast<int32_t>(ncol0), prob);
          }
          if (load_c) {
            if (!mbar_wait(cload_bar(epi_w, b), cphase[b], abort_flag, kFaultWaitCLoad, epi_w)) ok = false;
            cphase[b] ^= 1u;
          }
        } else {
          __syncwarp();  // previous plain write-out of this buffer is complete
          if (load_c) {
            // coalesced read of old C: lane = row inside the chunk, loop over columns
            const uint32_t mi = mrow0 + lane;
#pragma unroll 4
            for (uint32_t t = 0; t < 32; ++t) {
              const uint32_t nj = ncol0 + t;
              float v = 0.f;
              if (mi < p.m && nj < p.n) v = c_plain[(size_t)mi + (size_t)nj * p.ldc];
              gbuf[t * 32u + ((((lane >> 2) ^ (t & 7u)) << 2) | (lane & 3u))] = v;
            }
            __syncwarp();
          }
        }
#pragma unroll
        for (uint32_t j = 0; j < 8; ++j) {
          float4* addr = reinterpret_cast<float4*>(gbuf + lane * 32u + ((j ^ (lane & 7u)) << 2));
          float4 v = make_float4(alpha * sums[32 * c + 4 * j], alpha * sums[32 * c + 4 * j + 1],
                                 alpha * sums[32 * c + 4 * j + 2], alpha * sums[32 * c + 4 * j + 3]);
          if (load_c) {
            const float4 old = *addr;
            v.x = fmaf(beta, old.x, v.x);
            v.y = fmaf(beta, old.y, v.y);
            v.z = fmaf(beta, old.z, v.z);
            v.w = fmaf(beta, old.w, v.w);
          }
          *addr = v;
        }
        if (c_tma) {
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (in_range && ok)
              tma_store_tile(batched, &tmap_c, sbuf, static_cast<int32_t>(mrow0), static_cast<int32_t>(ncol0), prob);
            tma_store_commit();
          }
        } else {
          __syncwarp();
          if (in_range) {
            const uint32_t mi = mrow0 + lane;
#pragma unroll 4
            for (uint32_t t = 0; t < 32; ++t) {
              const uint32_t nj = ncol0 + t;
              const float v = gbuf[t * 32u + ((((lane >> 2) ^ (t & 7u)) << 2) | (lane & 3u))];
              if (mi < p.m && nj < p.n) c_plain[(size_t)mi + (size_t)nj * p.ldc] = v;
            }
          }
        }
        ok = __all_sync(0xffffffffu, ok);
      }
    }
    if (lane == 0) tma_store_wait_all<0>();
  }

  tcgen05_fence_before();
  __syncthreads();
  if constexpr (CG == 2) {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  }
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc<CG>(tmem_base, kTmemCols);
  }
}

}  // namespace mmbo
