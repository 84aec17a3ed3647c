// HGEMM (fp16 in, fp32 accumulate, fp16 out) on the sm_100a tensor cores:
//   C = alpha * op(A) * op(B) + beta * C      (column-major, BLAS op() convention)
//
// This is the B200 counterpart of the reference's device kernels (general path:
// src/gemm/ref/Kernels.cpp:153-1123; hand-tuned path:
// src/gemm/assembly/naive_gemm_kernel_MT096x096x08_TT06_06_STT02_06_WG16_16_01_HALF_A_HALF_B.s),
// redesigned around tcgen05:
//
//   * The kernel computes the transposed tile  D[n][m] = sum_l op(B)(l,n) * op(A)(m,l):
//     the UMMA "M" axis (128 tensor-memory lanes) runs along the problem's N and the
//     UMMA "N" axis (TM tensor-memory columns) runs along the problem's M, which is the
//     contiguous axis of column-major C.  An epilogue thread therefore owns one column
//     of C and TM consecutive rows of it, and packs 8 fp16 per 16-byte access.
//   * No operand is ever transposed in memory: NN/NT/TN/TT only change which tensor
//     map describes an operand and whether its shared-memory tile is "K-major"
//     (contraction index contiguous: transA = T, transB = N) or "MN-major".
//   * Roles: warp 0 = TMA producer (one elected lane), warp 1 = tensor memory owner +
//     UMMA issuer (one lane), then EW epilogue warps: one per 32-lane quarter of tensor
//     memory (192 threads), or two per quarter that split the columns (320 threads) for
//     shapes with a short contraction, where the epilogue is what bounds the kernel.
//   * STAGES-deep ring of 128-byte-swizzled shared-memory tiles fed by TMA; two
//     accumulators in tensor memory so the epilogue of tile i overlaps the main loop
//     of tile i+1 (the idea sketched by the reference's two-tiles-per-work-group kernel,
//     ..._HALF_A_HALF_B_ver3.s:931-962); persistent CTAs walk tiles in the reference's
//     work-group-mapping order (raster.h).
//   * Epilogue: tcgen05.ld -> alpha*acc (+ beta*C, with C fetched by TMA into the same
//     staging buffer; beta == 0 never reads C, src/gemm/ref/Kernels.cpp:87) -> fp16 ->
//     swizzled staging -> TMA store, per warp, double buffered.
//   * Ragged M, N, K need no special code on the load side: TMA zero-fills out-of-range
//     loads.  TMA stores clip out-of-range elements in units of 16 bytes, so C goes
//     through TMA only when m is a multiple of 8 (and C is 16-byte aligned with
//     ldc % 8 == 0); otherwise the epilogue writes its staging tile with coalesced plain
//     stores (and reads the old C the same way).
//
// Requirements checked by the host before choosing this kernel: A and B have 16-byte
// aligned bases and leading dimensions that are multiples of 8 elements (TMA strides).
#pragma once

#include <cuda_fp16.h>

#include <type_traits>

#include "ptx.cuh"
#include "raster.h"

// 512-row tiles keep the op(B) operand of a k-step's first UMMA in the tensor core's collector buffer for its
// second one, which then does not read shared memory for it (measured against a build without it: 8192^3
// 1412-1444 against 1406 TFLOP/s, seconds-long loops under the power cap 1289 against 1264).  Build with
// -DMMBO_COLLECTOR_A=0 to compare.
#ifndef MMBO_COLLECTOR_A
#define MMBO_COLLECTOR_A 1
#endif
// Probe builds only (-DMMBO_TRACE_KB=1): extra trace stamps inside the k loops of the producer and the issuer
// (slot 13/14: first/last operand stage of the tile has arrived; slot 15: the producer got the tile's first
// free stage).  Off in the shipped library: a branch in the issuer's loop costs throughput.
#ifndef MMBO_TRACE_KB
#define MMBO_TRACE_KB 0
#endif
// Probe build 3: per-role accounting of the cycles spent in barrier waits (totals written at the end of each
// role's loop to slots of trace tile 62).
#if MMBO_TRACE_KB == 3
#define MMBO_ACCT_BEGIN() const long long acct_t_ = clock64()
#define MMBO_ACCT_END(var) var += clock64() - acct_t_
#define MMBO_ACCT_OUT(slot, v) if (p.trace != nullptr && blockIdx.x == 0) p.trace[62 * 16 + (slot)] = (unsigned long long)(v)
#else
#define MMBO_ACCT_BEGIN()
#define MMBO_ACCT_END(var)
#define MMBO_ACCT_OUT(slot, v)
#endif

namespace mmbo {

constexpr int kTileN = 128;  // problem-N extent of a CTA tile = UMMA M
constexpr int kBlockK = 64;  // fp16 elements per stage along K = one 128-byte swizzle row
constexpr int kUmmaK = 16;   // K extent of one kind::f16 UMMA
constexpr int kEpiBufBytesMax = 32 * 128;  // 32 C columns x 64 rows of fp16: the larger of the two staging buffer sizes

// CG = CTAs cooperating on one UMMA (cta_group): 1, or 2 for a CTA pair that shares a
// 256-lane accumulator; each CTA of a pair stages its own 128 rows of op(B) and its own
// half (TM / 2 rows) of op(A).
// EW = epilogue warps: 4 (one per 32-lane quarter of tensor memory) or 8 (two per
// quarter, each taking half of the accumulator's columns).
// CSETS = sets of staging buffers per epilogue warp: 2 lets the old C of the next tile be requested a tile
// ahead (shared memory that then cannot hold operand stages), 1 keeps two buffers per warp and relies on
// an L2 prefetch of the next tile's C.
template <int TM, int STAGES, int CG = 1, int EW = 4, int CSETS = (EW == 8 ? 2 : 1)>
struct HgemmSmem {
  static constexpr int kThreads = 64 + 32 * EW;
  static constexpr int kAopRows = TM / CG;                // rows of op(A) staged by one CTA
  // One UMMA covers at most 256 rows of op(A).  A 512-row tile is two UMMAs per k-step on the same op(B)
  // operand, each on one "piece" of op(A): piece h holds this CTA's 128 rows of rows [256h, 256h + 256) of the
  // tile, so that accumulator columns map to tile rows in order.
  static constexpr int kPieceRows = TM == 512 ? 128 : kAopRows;
  static constexpr int kPieces = kAopRows / kPieceRows;
  static constexpr int kBopBytes = kTileN * kBlockK * 2;  // op(B) tile  (UMMA A operand)
  static constexpr int kAopBytes = kAopRows * kBlockK * 2;  // op(A) tile  (UMMA B operand)
  static constexpr int kStageBytes = kBopBytes + kAopBytes;
  static constexpr int kEpiOffset = STAGES * kStageBytes;
  // Staging buffers per epilogue warp: two; with 8 epilogue warps (at most two chunks per warp
  // and tile) two sets of two, so that the old C of the next tile can be requested a whole
  // tile ahead while this tile's set is still in use.
  static constexpr int kCSets = CSETS;
  static constexpr int kBufsPerWarp = 2 * kCSets;
  // Rows of C per epilogue chunk (a chunk = these rows x the warp's 32 columns, one staging buffer, one TMA
  // load of old C and one TMA store): 64 (128-byte staging rows, 128-byte swizzle), or 32 (64-byte rows, 64-byte
  // swizzle) where a 512-row tile gets eight epilogue warps -- half-size buffers keep their double buffering
  // inside the 32 KB that four warps with 64-row chunks take, next to four 48 KB operand stages.
  static constexpr int kChunkRows = (TM == 512 && EW == 8) ? 32 : 64;
  static constexpr int kBufBytes = 32 * kChunkRows * 2;
  static constexpr int kEpiBytes = EW * kBufsPerWarp * kBufBytes;
  static constexpr int kBarOffset = kEpiOffset + kEpiBytes;
  // Accumulators in tensor memory (512 columns): two of 256 columns, or four of 128 -- with short
  // contractions the deeper queue keeps the UMMA issuer from ever waiting for the epilogue.
  static constexpr int kAccs = 512 / TM;
  // full[STAGES], empty[STAGES], tmem_full[kAccs], tmem_empty[kAccs], cload[EW][kBufsPerWarp]
  static constexpr int kNumBars = 2 * STAGES + 2 * kAccs + kBufsPerWarp * EW;
  static constexpr int kMiscOffset = kBarOffset + kNumBars * 8;
  static constexpr int kTotal = kMiscOffset + 16;
  static constexpr int kDynamic = kTotal + 1024;  // slack to align the base to 1024 bytes
};

struct HgemmParams {
  uint32_t m, n, k;
  uint32_t tiles_m, tiles_n;  // ceil(m / TM), ceil(n / (128 * CG))
  uint32_t batch;             // problems of a strided batch (the reference's kernel takes its batch index
                              // from the grid: src/gemm/ref/Kernels.cpp:254); the persistent walk covers
                              // batch * tiles_m * tiles_n tiles, problem index slowest
  unsigned long long c_batch_stride;  // elements between the C of consecutive problems (plain epilogue)
  uint32_t wgm;               // work-group-mapping width (tile columns per block)
  MmboTileWalk walk;          // the same walk with its divisions precomputed (mmbo_tile_walk_make(tiles_m, tiles_n, wgm))
  float alpha, beta;
  __half* c;       // C and its leading dimension, for the epilogue without TMA
  uint32_t ldc;
  __half* c_mc;    // optional: a multicast address of the same C window (every GPU bound to it receives each
                   // store); when set, finished chunks are written there with multimem.st instead of the TMA store
  unsigned long long* trace;  // optional event trace (clock stamps of CTA 0), null in production
  uint32_t diag;   // diagnostic builds, results wrong by design (the reference keeps such
                   // kernels too: test_main_loop.s has no C store, error_kernel_000.s no waits):
                   // bit 0 = no C store, bit 1 = no tensor-memory drain either
  uint32_t c_tma;  // 1: C goes through the tensor map (16-byte aligned base, ldc % 8 == 0,
                   // m % 8 == 0: TMA stores whole 16-byte units, so a ragged m would spill
                   // into the padding rows below the matrix)
};

// Destinations beyond C itself: the same window of C in the memory of other GPUs of the node
// (peer mappings).  The epilogue stores every finished chunk to each of them with one more TMA
// store from the same staging buffer, so that a column-sharded GEMM leaves the assembled
// matrix on every GPU without a separate all-gather (stores only: nothing is ever loaded
// through these maps).
constexpr int kMaxPeerCopies = 7;
struct alignas(64) HgemmPeerMaps {
  CUtensorMap map[kMaxPeerCopies];
  uint32_t count;
  uint32_t pad[15];
};

__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Event trace for performance work: when HgemmParams::trace is set, the UMMA issuer and
// the first epilogue warp of CTA 0 record clock stamps per tile (16 slots per tile:
// 0-7 epilogue, 8-15 issuer).  The counterpart of the reference's #ifdef DEBUG prints
// (src/gemm/driver.h:38-55), for the device side.
__device__ __forceinline__ void trace_stamp(unsigned long long* trace, uint32_t tile_slot, uint32_t ev) {
#if MMBO_TRACE_KB >= 2
  if (tile_slot != 63u) return;  // probe build: only the launch-level stamps (kernel entry, loops done, exit)
#endif
  if (trace != nullptr && blockIdx.x == 0 && tile_slot < 64u) trace[tile_slot * 16u + ev] = clock64();
}

template <int TM, int STAGES, bool A_KMAJOR, bool B_KMAJOR, int CG = 1, int EW = 4, int CSETS = (EW == 8 ? 2 : 1)>
__global__ void __launch_bounds__(64 + 32 * EW, 1)
hgemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a,
                     const __grid_constant__ CUtensorMap tmap_b,
                     const __grid_constant__ CUtensorMap tmap_c, const HgemmParams p,
                     const __grid_constant__ HgemmPeerMaps peers) {
  using L = HgemmSmem<TM, STAGES, CG, EW, CSETS>;
  static_assert(TM == 128 || TM == 256 || (TM == 512 && CG == 2), "128 or 256 rows per UMMA; 512 = two UMMAs per k-step of a CTA pair");
  static_assert(EW == 4 || EW == 8, "one or two epilogue warps per tensor-memory quarter");
  // 64-row chunks of the accumulator each epilogue warp drains per tile
  constexpr uint32_t kCR = L::kChunkRows;              // rows of C per chunk
  constexpr uint32_t kEpiBufBytes = L::kBufBytes;      // one staging buffer
  constexpr uint32_t kRowPieces = kCR / 8u;            // 16-byte pieces per staging row (one C column of a chunk)
  constexpr uint32_t kLdPerChunk = kCR / 32u;          // 32-column tensor-memory loads per chunk
  constexpr uint32_t kChunksPerWarp = (TM / kCR) / (EW / 4);
  // 16-byte piece j of staging row t lives at piece swz(j, t): the TMA swizzle of the C tensor map (128-byte
  // rows: j ^ (t & 7); 64-byte rows: j ^ ((t >> 1) & 3)).
  auto swz = [](uint32_t j, uint32_t t) -> uint32_t { return kCR == 64u ? (j ^ (t & 7u)) : (j ^ ((t >> 1) & 3u)); };
  static_assert(kChunksPerWarp >= 1, "tile too narrow for this many epilogue warps");
  static_assert(CG == 1 || CG == 2, "one CTA or a CTA pair per UMMA");
  constexpr uint32_t kAccs = L::kAccs;
  constexpr uint32_t kTmemCols = kAccs * TM;  // = 512: all of tensor memory
  // CTA pair: rank 0 (the leader) issues every UMMA and owns the barriers that count
  // both CTAs' copies; this CTA's index among the tile walkers is its cluster's index.
  const uint32_t cta_rank = (CG == 2) ? cluster_cta_rank() : 0u;
  const uint32_t walker = blockIdx.x / CG;
  const uint32_t num_walkers = gridDim.x / CG;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
#if MMBO_TRACE_KB
  if (threadIdx.x == 0) {
    trace_stamp(p.trace, 63u, 0);
    if (p.trace != nullptr && blockIdx.x == 0) p.trace[63 * 16 + 6] = global_timer_ns();
  }
#endif

  const uint32_t bar_base = smem_base + L::kBarOffset;
  auto full_bar = [&](uint32_t s) { return bar_base + 8u * s; };
  auto empty_bar = [&](uint32_t s) { return bar_base + 8u * (STAGES + s); };
  auto tmem_full_bar = [&](uint32_t a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tmem_empty_bar = [&](uint32_t a) { return bar_base + 8u * (2 * STAGES + kAccs + a); };
  auto cload_bar = [&](uint32_t w, uint32_t b) { return bar_base + 8u * (2 * STAGES + 2 * kAccs + L::kBufsPerWarp * w + b); };
  volatile uint32_t* tmem_ptr_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kMiscOffset);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kMiscOffset + 4);

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t tiles_per_problem = p.tiles_m * p.tiles_n;
  const uint32_t num_tiles = tiles_per_problem * p.batch;
  const uint32_t num_kb = (p.k + kBlockK - 1) / kBlockK;
  // tile id of the walk -> (tile row, tile column, problem of the batch)
  const bool batched = p.batch > 1u;  // 3-D tensor maps; single problems keep the 2-D forms
  auto locate = [&](uint32_t tile, uint32_t* tm, uint32_t* tn) -> uint32_t {
    const uint32_t prob = batched ? mmbo_fastdiv(tile, p.walk.by_problem) : 0u;
    mmbo_tile_walk_locate(p.walk, tile - prob * tiles_per_problem, tm, tn);
    return prob;
  };

  // ------------------------------------------------------------------ set-up --------
  static_assert(L::kNumBars <= L::kThreads, "one thread per barrier");
  if (threadIdx.x < (uint32_t)L::kNumBars) {
    // one barrier per thread: a single arrival everywhere except on the accumulator-empty barriers, where
    // every epilogue warp of the CTA (pair) arrives
    const uint32_t i = threadIdx.x;
    const bool acc_empty = i >= 2u * STAGES + kAccs && i < 2u * STAGES + 2u * kAccs;
    mbar_init(bar_base + 8u * i, acc_empty ? EW * CG : 1);
    fence_mbar_init();
  }
  if (threadIdx.x == 0) {
    *abort_flag = 0u;
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
    if (p.c_tma) prefetch_tensormap(&tmap_c);
  }
  __syncwarp();
  if (warp == 1) {
    tmem_alloc<CG>(smem_u32(const_cast<uint32_t*>(tmem_ptr_slot)), kTmemCols);
    tmem_relinquish<CG>();
  }
  tcgen05_fence_before();
  __syncthreads();
  if constexpr (CG == 2) cluster_sync_all();  // peer's barriers and tensor memory are ready
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_ptr_slot;
#if MMBO_TRACE_KB
  if (threadIdx.x == 0) trace_stamp(p.trace, 63u, 1);
#endif
  // Set-up is done without touching global memory: the next kernel of the stream may start its own set-up now,
  // and this one goes on only when the kernel before it has completed (its C may be this one's operand).
  griddep_launch_dependents();
  griddep_wait();

  // ------------------------------------------------------------------ roles ---------
  if (warp == 0) {
    // ===== TMA producer =====
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, issued = 0;
      bool ok = true;
      [[maybe_unused]] long long w_empty = 0;
      [[maybe_unused]] const long long loop_t0 = clock64();
      for (uint32_t tile = walker; ok && tile < num_tiles; tile += num_walkers) {
        uint32_t tm_idx, tn_idx;
        const int32_t prob = static_cast<int32_t>(locate(tile, &tm_idx, &tn_idx));
        // This CTA's share of the tile: its own 128 columns of C (rows of op(B)^T) and
        // its own TM / CG rows of op(A).
        // piece h of op(A): this CTA's kPieceRows rows of the h-th 256-row (or whole) part of the tile
        const int32_t m0 = static_cast<int32_t>(tm_idx * TM + cta_rank * L::kPieceRows);
        constexpr int32_t kPieceStep = L::kPieceRows * CG;
        const int32_t n0 = static_cast<int32_t>((tn_idx * CG + cta_rank) * kTileN);
        for (uint32_t kb = 0; kb < num_kb; ++kb) {
          MMBO_ACCT_BEGIN();
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, kFaultWaitEmpty, stage)) {
            ok = false;
            break;
          }
          MMBO_ACCT_END(w_empty);
#if MMBO_TRACE_KB
          if (kb == 0) trace_stamp(p.trace, (tile - walker) / num_walkers, 15);
#endif
          // Completion is counted on the leader's barrier, which expects both CTAs' bytes.
          const uint32_t bar = (CG == 2) ? mapa_shared(full_bar(stage), 0u) : full_bar(stage);
          const uint32_t s_bop = smem_base + stage * L::kStageBytes;
          const uint32_t s_aop = s_bop + L::kBopBytes;
          const int32_t k0 = static_cast<int32_t>(kb * kBlockK);
#if MMBO_TRACE_KB
          // probe builds: no operand loads after the first fill of the ring (the UMMAs run on what the stages hold;
          // bit 3 set: no loads at all, the stages stay as they were found)
          if ((p.diag & 4u) && (issued >= STAGES || (p.diag & 8u))) {
            if (cta_rank == 0) mbar_arrive(full_bar(stage));
            ++issued;
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1u;
            }
            continue;
          }
#endif
          if (cta_rank == 0) mbar_expect_tx(full_bar(stage), L::kStageBytes * CG);
          auto load = [&](uint32_t dst, const CUtensorMap* map, int32_t c0, int32_t c1) {
            if constexpr (CG == 2) tma_load_tile_pair(batched, dst, map, bar, c0, c1, prob);
            else tma_load_tile(batched, dst, map, bar, c0, c1, prob);
          };
          if constexpr (B_KMAJOR) {
            load(s_bop, &tmap_b, k0, n0);  // box {64 k, 128 n}
          } else {
#pragma unroll
            for (int c = 0; c < kTileN / 64; ++c)  // boxes {64 n, 64 k}
              load(s_bop + c * 8192, &tmap_b, n0 + 64 * c, k0);
          }
#pragma unroll
          for (int h = 0; h < L::kPieces; ++h) {
            const uint32_t s_piece = s_aop + h * (L::kPieceRows * kBlockK * 2);
            const int32_t mp = m0 + h * kPieceStep;
            if constexpr (A_KMAJOR) {
              load(s_piece, &tmap_a, k0, mp);  // box {64 k, kPieceRows m}
            } else {
#pragma unroll
              for (int c = 0; c < L::kPieceRows / 64; ++c)  // boxes {64 m, 64 k}
                load(s_piece + c * 8192, &tmap_a, mp + 64 * c, k0);
            }
          }
          ++issued;
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      MMBO_ACCT_OUT(0, clock64() - loop_t0);
      MMBO_ACCT_OUT(1, w_empty);
      if (!ok && cta_rank == 0) {
        // Unwind: let every copy this thread issued land before the CTA's shared
        // memory is released.  A stage already consumed reports complete at once.
        // (In a CTA pair the leader's barriers count both CTAs' copies, and neither CTA
        // leaves before the cluster barrier at the end of the kernel.)
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
    // ===== UMMA issuer (leader CTA of a pair) =====
    if (lane == 0 && cta_rank == 0) {
      constexpr uint32_t kUmmaN = TM < 256 ? TM : 256;  // accumulator columns one UMMA writes
      constexpr uint32_t idesc = make_idesc(0u, B_KMAJOR ? 0u : 1u, A_KMAJOR ? 0u : 1u, kTileN * CG, kUmmaN);
      constexpr uint32_t kStepBop = B_KMAJOR ? 32u : 2048u;  // bytes per UMMA K step
      constexpr uint32_t kStepAop = A_KMAJOR ? 32u : 2048u;
      constexpr uint32_t kLboBop = B_KMAJOR ? 16u : 8192u;
      constexpr uint32_t kLboAop = A_KMAJOR ? 16u : 8192u;
      uint32_t stage = 0, phase = 0, local_tile = 0;
      bool ok = true;
      [[maybe_unused]] long long w_acc = 0, w_full = 0;
      [[maybe_unused]] const long long loop_t0 = clock64();
      for (uint32_t tile = walker; ok && tile < num_tiles; tile += num_walkers, ++local_tile) {
        const uint32_t acc = local_tile % kAccs;
        const uint32_t acc_phase = (local_tile / kAccs) & 1u;
        trace_stamp(p.trace, local_tile, 8);
        {
          MMBO_ACCT_BEGIN();
          if (!mbar_wait(tmem_empty_bar(acc), acc_phase ^ 1u, abort_flag, kFaultWaitTmemEmpty, acc)) {
            ok = false;
            break;
          }
          MMBO_ACCT_END(w_acc);
        }
        trace_stamp(p.trace, local_tile, 9);
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc * TM;
        for (uint32_t kb = 0; kb < num_kb; ++kb) {
          {
            MMBO_ACCT_BEGIN();
            if (!mbar_wait(full_bar(stage), phase, abort_flag, kFaultWaitFull, stage)) {
              ok = false;
              break;
            }
            MMBO_ACCT_END(w_full);
          }
          tcgen05_fence_after();
#if MMBO_TRACE_KB
          if (kb == 0) trace_stamp(p.trace, local_tile, 13);
          if (kb + 1 == num_kb) trace_stamp(p.trace, local_tile, 14);
#endif
          const uint32_t s_bop = smem_base + stage * L::kStageBytes;
          const uint32_t s_aop = s_bop + L::kBopBytes;
          const uint64_t desc_a = make_smem_desc_sw128(s_bop, kLboBop, 1024u);
          const uint64_t desc_b = make_smem_desc_sw128(s_aop, kLboAop, 1024u);
#pragma unroll
          for (uint32_t j = 0; j < kBlockK / kUmmaK; ++j) {
#pragma unroll
            for (uint32_t h = 0; h < (uint32_t)L::kPieces; ++h) {  // one UMMA per 256-row piece, same op(B) operand
              const uint64_t piece = (uint64_t)((h * (uint32_t)(L::kPieceRows * kBlockK * 2)) >> 4);
              const uint64_t da = desc_a + ((j * kStepBop) >> 4), db = desc_b + piece + ((j * kStepAop) >> 4);
              const uint32_t accumulate = (kb | j) != 0u ? 1u : 0u;
              if constexpr (MMBO_COLLECTOR_A != 0 && L::kPieces == 2 && CG == 2) {
                // the second UMMA of the pair takes op(B) from the collector buffer
                if (h == 0) umma_ss_pair_f16_collect_a<false>(d_tmem, da, db, idesc, accumulate);
                else umma_ss_pair_f16_collect_a<true>(d_tmem + kUmmaN, da, db, idesc, accumulate);
              } else {
                umma_ss<CG, false>(d_tmem + h * kUmmaN, da, db, idesc, accumulate);
              }
            }
          }
          // frees the stage (in both CTAs of a pair) once these UMMAs have read it
          if constexpr (CG == 2) umma_commit_pair(empty_bar(stage), 3);
          else umma_commit(empty_bar(stage));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        trace_stamp(p.trace, local_tile, 10);
        if (ok) {  // accumulator complete (in both CTAs of a pair)
          if constexpr (CG == 2) umma_commit_pair(tmem_full_bar(acc), 3);
          else umma_commit(tmem_full_bar(acc));
        }
      }
#if MMBO_TRACE_KB
      trace_stamp(p.trace, 63u, 2);
#endif
      MMBO_ACCT_OUT(2, clock64() - loop_t0);
      MMBO_ACCT_OUT(3, w_acc);
      MMBO_ACCT_OUT(4, w_full);
    }
    __syncwarp();
  } else {
    // ===== epilogue: warp owns tensor-memory lanes [32q, 32q+32) = 32 columns of C, and
    // kChunksPerWarp 64-row chunks of them (all of them with 4 warps, half with 8) =====
    const uint32_t q = warp & 3u;
    const uint32_t epi_w = warp - 2u;
    const uint32_t col_base = (epi_w >> 2) * kChunksPerWarp * kCR;  // first accumulator column of this warp
    const uint32_t warp_buf_base = smem_base + L::kEpiOffset + epi_w * L::kBufsPerWarp * kEpiBufBytes;
    uint8_t* warp_buf_gen = smem_gen + L::kEpiOffset + epi_w * L::kBufsPerWarp * kEpiBufBytes;
    const bool use_c = (p.beta != 0.0f);
    const bool c_tma = p.c_tma != 0u;
    const float alpha = p.alpha, beta = p.beta;
    const uint64_t alpha2 = pack_f32x2(__float_as_uint(alpha), __float_as_uint(alpha));
    const uint64_t beta2 = pack_f32x2(__float_as_uint(beta), __float_as_uint(beta));
    const bool alpha_one = alpha == 1.0f;
    uint32_t local_tile = 0;
    uint32_t cphase = 0;  // bit b: phase parity of the load barrier of buffer b
    bool ok = true;
    // With two buffer sets the old C of tile i + 1 is requested at the start of tile i (into
    // the set tile i - 1 used), so that its HBM latency hides behind a whole tile.
    constexpr bool kCAhead = L::kCSets == 2;
    static_assert(!kCAhead || kChunksPerWarp <= 2, "C one tile ahead needs a buffer per chunk");
    // The warp's staging buffers form kSets sets of kSetChunks (one per chunk of a tile); tile i uses set
    // i % kSets.  With several sets the old C of tile i + kSets - 1 is requested during tile i (into the set
    // tile i - 1 used), so that its HBM latency hides behind kSets - 1 whole tiles: one tile ahead with
    // 256-row tiles (two sets of two), three tiles ahead with 128-row tiles (four sets of one).
    constexpr uint32_t kSetChunks = kChunksPerWarp < 2u ? kChunksPerWarp : 2u;
    constexpr uint32_t kSets = kCAhead ? (uint32_t)L::kBufsPerWarp / kSetChunks : 1u;
    constexpr uint32_t kAhead = kSets - 1u;
    constexpr int kStoresPending = (int)(kSets * kSetChunks) - 1;  // bulk groups that may still be reading other buffers
    [[maybe_unused]] long long w_tfull = 0, w_cload = 0, w_store = 0, w_rel = 0;
    [[maybe_unused]] const long long loop_t0 = clock64();
    uint32_t c_in_flight = 0;  // bit b: a load into buffer b of this warp has been requested and not yet awaited
    auto request_c = [&](uint32_t t, uint32_t set) {  // whole warp; lane 0 issues: chunks of tile t into buffer set `set`
      uint32_t tm, tn;
      const int32_t pr = static_cast<int32_t>(locate(t, &tm, &tn));
      const uint32_t mr = tm * TM + col_base, nc = (tn * CG + cta_rank) * kTileN + 32u * q;
#pragma unroll
      for (uint32_t c = 0; c < kSetChunks; ++c) {
        const uint32_t mrow0 = mr + kCR * c;
        if (mrow0 < p.m && nc < p.n) {
          c_in_flight |= 1u << (kSetChunks * set + c);
          if (lane == 0) {
            mbar_expect_tx(cload_bar(epi_w, kSetChunks * set + c), kEpiBufBytes);
            tma_load_tile(batched, warp_buf_base + (kSetChunks * set + c) * kEpiBufBytes, &tmap_c, cload_bar(epi_w, kSetChunks * set + c),
                        static_cast<int32_t>(mrow0), static_cast<int32_t>(nc), pr);
          }
        }
      }
    };
    if (kCAhead && p.c_tma != 0u && use_c) {
#pragma unroll
      for (uint32_t a = 0; a < kAhead; ++a)
        if (walker + a * num_walkers < num_tiles) request_c(walker + a * num_walkers, a);
    }
    for (uint32_t tile = walker; ok && tile < num_tiles; tile += num_walkers, ++local_tile) {
      uint32_t tm_idx, tn_idx;
      const int32_t prob = static_cast<int32_t>(locate(tile, &tm_idx, &tn_idx));
      __half* const c_plain = p.c + static_cast<size_t>(prob) * p.c_batch_stride;  // this problem's C (plain epilogue)
      const uint32_t m0 = tm_idx * TM + col_base;
      const uint32_t ncol0 = (tn_idx * CG + cta_rank) * kTileN + 32u * q;  // first C column of this warp
      const uint32_t acc = local_tile % kAccs;
      const uint32_t acc_phase = (local_tile / kAccs) & 1u;
      // Staging tile b (two per warp): row t = C column ncol0 + t, 64 fp16 = C rows of one
      // chunk; the 16-byte piece j of a row lives at piece j ^ (t & 7) (128-byte TMA swizzle).
      // With beta != 0 the old C of the first two chunks is requested now, before the wait
      // for the accumulator, so that its latency overlaps the main loop of this tile.
      const bool tracer = (warp == 2u && lane == 0u);
      if (tracer) trace_stamp(p.trace, local_tile, 0);
      // buffer set of this tile
      const uint32_t set = (kCAhead && c_tma) ? local_tile % kSets : 0u;
      const uint32_t buf_base = warp_buf_base + kSetChunks * set * kEpiBufBytes;
      uint8_t* buf_gen = warp_buf_gen + kSetChunks * set * kEpiBufBytes;
      if (!kCAhead && c_tma && use_c) {
        if (lane == 0) tma_store_wait_read<0>();  // the previous tile's stores have read their buffers
        __syncwarp();
        request_c(tile, 0u);
      }
      if (tracer) trace_stamp(p.trace, local_tile, 1);
      // ... and the old C of the tile after this one is pulled into L2 now, one whole tile
      // ahead, so that those requests will not have to go to HBM.
      if (!kCAhead && c_tma && use_c && lane == 0 && tile + num_walkers < num_tiles) {
        uint32_t nm, nn;
        const int32_t npr = static_cast<int32_t>(locate(tile + num_walkers, &nm, &nn));
        const uint32_t nm0 = nm * TM + col_base, nn0 = (nn * CG + cta_rank) * kTileN + 32u * q;
#pragma unroll
        for (uint32_t c = 0; c < kChunksPerWarp; ++c)
          if (nm0 + kCR * c < p.m && nn0 < p.n)
            tma_prefetch_l2_tile(batched, &tmap_c, static_cast<int32_t>(nm0 + kCR * c), static_cast<int32_t>(nn0), npr);
      }
      // One lane polls (with back-off once the wait has become a long one); the outcome is warp-uniform so
      // that the aligned tcgen05 instructions below always run with a converged warp.
      {
        MMBO_ACCT_BEGIN();
        ok = mbar_wait_warp(tmem_full_bar(acc), acc_phase, abort_flag, kFaultWaitTmemFull, acc);
        MMBO_ACCT_END(w_tfull);
      }
      if (!ok) break;
      if (tracer) trace_stamp(p.trace, local_tile, 2);
      tcgen05_fence_after();
      const uint32_t t_warp = tmem_base + ((32u * q) << 16) + acc * TM + col_base;
      const bool drain = (p.diag & 2u) == 0u;
      auto release_accumulator = [&]() {
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) {
          if constexpr (CG == 2) mbar_arrive_cluster(mapa_shared(tmem_empty_bar(acc), 0u));
          else mbar_arrive(tmem_empty_bar(acc));
        }
      };
      // With at most 128 accumulator columns per warp the whole share is pulled into registers (no
      // register buffer is reused within a tile) and the accumulator handed back at once: a 32-column
      // tensor-memory load takes about 17 cycles once the loads are pipelined (86 cycles for 128 columns; the
      // two warps of a scheduler share its port), so the hand-back comes a few hundred cycles after the
      // accumulator is complete and the issuer can start the tile after next.
      constexpr bool kEarlyDrain = kChunksPerWarp <= 2;
      // Otherwise two register buffers of one chunk each: the tensor-memory loads of chunk
      // c + 1 are in flight while chunk c is scaled, converted and staged.
      uint32_t racc[kEarlyDrain ? 2 * kChunksPerWarp : 4][32];
      auto load_chunk = [&](const uint32_t c, uint32_t (&lo)[32], uint32_t (&hi)[32]) {
        if (drain) {
          tmem_ld_32x32(t_warp + kCR * c, lo);
          if constexpr (kLdPerChunk == 2) tmem_ld_32x32(t_warp + kCR * c + 32u, hi);
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) lo[e] = hi[e] = 0u;
        }
      };
      static_assert(kCR == 64u || !(kChunksPerWarp <= 2), "32-row chunks use the double-buffered drain");
      if constexpr (kEarlyDrain) {
        auto load_piece = [&](uint32_t i) {
          if (drain) tmem_ld_32x32(t_warp + 32u * i, racc[i]);
          else {
#pragma unroll
            for (int e = 0; e < 32; ++e) racc[i][e] = 0u;
          }
        };
        {
          MMBO_ACCT_BEGIN();
#pragma unroll
          for (uint32_t i = 0; i < 2 * kChunksPerWarp; ++i) load_piece(i);
          tmem_ld_wait();
          release_accumulator();
          MMBO_ACCT_END(w_rel);
        }
        if (tracer) trace_stamp(p.trace, local_tile, 3);
        if (kCAhead && c_tma && use_c && tile + kAhead * num_walkers < num_tiles) {
          // The set tile i - 1 used was last read by that tile's stores, issued a drain ago: by now
          // they have long left shared memory, so this wait does not stall.
          if (lane == 0) tma_store_wait_read<0>();
          __syncwarp();
          request_c(tile + kAhead * num_walkers, (local_tile + kAhead) % kSets);
        }
      }
      if constexpr (!kEarlyDrain) load_chunk(0u, racc[0], racc[1]);
      auto do_chunk = [&](const uint32_t c, auto parity) {
        constexpr uint32_t kPb = decltype(parity)::value;  // register buffer of this chunk (non-early drain)
        const uint32_t b = c & 1u;
        const uint32_t sbuf = buf_base + b * kEpiBufBytes;
        uint8_t* gbuf = buf_gen + b * kEpiBufBytes;
        const uint32_t mrow0 = m0 + kCR * c;
        const bool in_range = (mrow0 < p.m) && (ncol0 < p.n);  // warp-uniform
        const bool load_c = use_c && in_range;
        if (c_tma) {
          if (!use_c || c >= 2u) {
            // The store last issued from this buffer (kStoresPending + 1 chunks ago) must have read it.
            {
              MMBO_ACCT_BEGIN();
              if (lane == 0) tma_store_wait_read<kStoresPending>();
              __syncwarp();
              MMBO_ACCT_END(w_store);
            }
            if (load_c) c_in_flight |= 1u << (kSetChunks * set + b);
            if (load_c && lane == 0) {  // chunks beyond the two requested up front
              mbar_expect_tx(cload_bar(epi_w, kSetChunks * set + b), kEpiBufBytes);
              tma_load_tile(batched, sbuf, &tmap_c, cload_bar(epi_w, kSetChunks * set + b), static_cast<int32_t>(mrow0),
                          static_cast<int32_t>(ncol0), prob);
            }
          }
        } else {
          __syncwarp();  // the previous plain write-out of this buffer is complete
          if (load_c) {
            // coalesced read of the old C: lanes run along the rows of the chunk
            __half* hb = reinterpret_cast<__half*>(gbuf);
#pragma unroll 2
            for (uint32_t t = 0; t < 32; ++t) {
              const uint32_t nj = ncol0 + t;
#pragma unroll
              for (uint32_t hh = 0; hh < kLdPerChunk; ++hh) {
                const uint32_t i = lane + 32u * hh, mi = mrow0 + i;
                __half v = __float2half_rn(0.f);
                if (mi < p.m && nj < p.n) v = c_plain[(size_t)mi + (size_t)nj * p.ldc];
                hb[t * kCR + ((swz(i >> 3, t) << 3) | (i & 7u))] = v;
              }
            }
            __syncwarp();
          }
        }
        if (c_tma && load_c) {
          MMBO_ACCT_BEGIN();
          if (!mbar_wait(cload_bar(epi_w, kSetChunks * set + b), (cphase >> (kSetChunks * set + b)) & 1u, abort_flag,
                         kFaultWaitCLoad, epi_w))
            ok = false;
          MMBO_ACCT_END(w_cload);
          cphase ^= 1u << (kSetChunks * set + b);
          c_in_flight &= ~(1u << (kSetChunks * set + b));
        }
        if (tracer && c == 0) trace_stamp(p.trace, local_tile, 4);  // old C of chunk 0 has arrived
        // `ok` may differ between lanes only after a time-out, when the data is
        // discarded anyway; keep the warp converged for the aligned tcgen05 ops.
        if constexpr (!kEarlyDrain) {
          tmem_ld_wait();  // this chunk is in registers (nothing else is in flight)
          if (c + 1 < kChunksPerWarp) load_chunk(c + 1, racc[2 * (kPb ^ 1u)], racc[2 * (kPb ^ 1u) + 1]);
          else release_accumulator();  // this warp's part of the accumulator is read: hand it back
        }
        // alpha * acc (+ beta * old C) on pairs of fp32 values (fma.rn.f32x2: one instruction per pair, each
        // half rounded as the scalar operation would be), then one conversion per pair.  The two run-time
        // choices (old C or not, alpha == 1 or not) are made once per chunk, outside the unrolled loops:
        // with short contractions the epilogue warps are bound by instruction issue.
        auto convert = [&](auto with_c, auto scale) {
          constexpr bool kWithC = decltype(with_c)::value, kScale = decltype(scale)::value;
          uint8_t* const row = gbuf + lane * (2u * kCR);
#pragma unroll
          for (uint32_t h = 0; h < kLdPerChunk; ++h) {
            const uint32_t(&r)[32] = racc[kEarlyDrain ? 2 * c + h : 2 * kPb + h];
#pragma unroll
            for (uint32_t jj = 0; jj < 4; ++jj) {
              const uint32_t j = 4u * h + jj;  // 16-byte piece of the 128-byte row
              uint4* const addr = reinterpret_cast<uint4*>(row + (swz(j, lane) << 4));
              uint4 out, old;
              uint32_t* po = reinterpret_cast<uint32_t*>(&out);
              if constexpr (kWithC) old = *addr;
              const uint32_t* oldw = reinterpret_cast<const uint32_t*>(&old);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                uint64_t v = pack_f32x2(r[8 * jj + 2 * e], r[8 * jj + 2 * e + 1]);
                if constexpr (kScale) v = mul_f32x2(alpha2, v);
                if constexpr (kWithC) v = fma_f32x2(beta2, half2_to_f32x2(oldw[e]), v);
                po[e] = f32x2_to_half2(v);
              }
              *addr = out;
            }
          }
        };
        using Yes = std::true_type;
        using No = std::false_type;
        if (load_c) {
          if (alpha_one) convert(Yes{}, No{});
          else convert(Yes{}, Yes{});
        } else {
          if (alpha_one) convert(No{}, No{});
          else convert(No{}, Yes{});
        }
        if (tracer && c == 0) trace_stamp(p.trace, local_tile, 11);  // chunk 0 written to staging
        if (c_tma && p.c_mc != nullptr) {
          // One store per 16-byte piece to the multicast address of C: NVSwitch delivers it to every GPU
          // bound to that address, this one included, so the chunk crosses this GPU's links once however
          // many GPUs receive it.  Eight lanes cover the 128 contiguous bytes of one column piece.
          __syncwarp();
          if (in_range && ok && (p.diag & 1u) == 0u) {
#pragma unroll
            for (uint32_t i = 0; i < kRowPieces; ++i) {  // kRowPieces lanes per column, 32 / kRowPieces columns per pass
              const uint32_t t = lane / kRowPieces + (32u / kRowPieces) * i, j = lane % kRowPieces;
              const uint4 v = *reinterpret_cast<const uint4*>(gbuf + t * (2u * kCR) + (swz(j, t) << 4));
              const uint32_t row = mrow0 + 8u * j, col = ncol0 + t;
              if (row < p.m && col < p.n) multimem_st_v4(p.c_mc + (size_t)row + (size_t)col * p.ldc, v);
            }
          }
          fence_proxy_async_smem();  // the next writer of this buffer may be a TMA load of old C
          __syncwarp();
        } else if (c_tma) {
          fence_proxy_async_smem();
          __syncwarp();
          if (tracer && c == 0) trace_stamp(p.trace, local_tile, 12);  // fenced
          if (lane == 0) {
            if (in_range && ok && (p.diag & 1u) == 0u) {
              tma_store_tile(batched, &tmap_c, sbuf, static_cast<int32_t>(mrow0), static_cast<int32_t>(ncol0), prob);
              for (uint32_t d = 0; d < peers.count; ++d)  // the same chunk into every peer's copy of C (single problems only)
                tma_store_2d(&peers.map[d], sbuf, static_cast<int32_t>(mrow0), static_cast<int32_t>(ncol0));
            }
            tma_store_commit();  // one group: the buffer is free again when all of them have read it
          }
        } else {
          __syncwarp();
          if (in_range && (p.diag & 1u) == 0u) {
            const __half* hb = reinterpret_cast<const __half*>(gbuf);
#pragma unroll 2
            for (uint32_t t = 0; t < 32; ++t) {
              const uint32_t nj = ncol0 + t;
#pragma unroll
              for (uint32_t hh = 0; hh < kLdPerChunk; ++hh) {
                const uint32_t i = lane + 32u * hh, mi = mrow0 + i;
                const __half v = hb[t * kCR + ((swz(i >> 3, t) << 3) | (i & 7u))];
                if (mi < p.m && nj < p.n) c_plain[(size_t)mi + (size_t)nj * p.ldc] = v;
              }
            }
          }
        }
        if (tracer) trace_stamp(p.trace, local_tile, 5 + (c == 0 ? 0 : 1));
        ok = __all_sync(0xffffffffu, ok);
      };
      using P0 = std::integral_constant<uint32_t, 0>;
      using P1 = std::integral_constant<uint32_t, 1>;
      if constexpr (kEarlyDrain) {  // unrolled: the register copy of the accumulator is indexed statically
#pragma unroll
        for (uint32_t c = 0; c < kChunksPerWarp; ++c) do_chunk(c, P0{});
      } else {
        static_assert(kEarlyDrain || kChunksPerWarp % 2 == 0, "chunks are taken in pairs");
#pragma unroll 1
        for (uint32_t c = 0; c < kChunksPerWarp; c += 2) {
          do_chunk(c, P0{});
          do_chunk(c + 1, P1{});
        }
      }
    }
    if (!ok) {
      // After a time-out: leave only when the loads of old C still in flight have landed
      // (a short bounded wait per buffer).
      for (uint32_t b = 0; b < (uint32_t)L::kBufsPerWarp; ++b) {
        if (c_in_flight & (1u << b)) {
          const uint64_t t0 = global_timer_ns();
          while (!mbar_try_wait(cload_bar(epi_w, b), (cphase >> b) & 1u) && global_timer_ns() - t0 < MMBO_DRAIN_LIMIT_NS) {
          }
        }
      }
    }
#if MMBO_TRACE_KB
    if (warp == 2u && lane == 0u) trace_stamp(p.trace, 63u, 3);
#endif
    if (warp == 2u && lane == 0u) {
      MMBO_ACCT_OUT(5, clock64() - loop_t0);
      MMBO_ACCT_OUT(6, w_tfull);
      MMBO_ACCT_OUT(7, w_cload);
      MMBO_ACCT_OUT(8, w_store);
      MMBO_ACCT_OUT(9, w_rel);
    }
    // Shared memory only has to outlive the stores' reads of it; the end of the grid makes their writes visible.
    if (lane == 0) tma_store_wait_read<0>();
#if MMBO_TRACE_KB
    if (warp == 2u && lane == 0u) trace_stamp(p.trace, 63u, 4);
#endif
  }

  // ------------------------------------------------------------------ teardown ------
  tcgen05_fence_before();
  __syncthreads();
  // A CTA of a pair must outlive every access its peer makes to its shared memory,
  // barriers and tensor memory.
  if constexpr (CG == 2) cluster_sync_all();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc<CG>(tmem_base, kTmemCols);
  }
#if MMBO_TRACE_KB
  if (threadIdx.x == 0) {
    trace_stamp(p.trace, 63u, 5);
    if (p.trace != nullptr && blockIdx.x == 0) p.trace[63 * 16 + 7] = global_timer_ns();
  }
#endif
}

}  // namespace mmbo
