// Stream-K work split for the persistent producer / consumer kernels (fp64 tensor kernel, fp32
// FFMA kernel): the contraction of the whole problem is cut into (tile, k-slab) units and every
// CTA takes one contiguous run of units, so that a problem whose tile count does not fill whole
// rounds of the resident CTAs still keeps every CTA busy to the end.  The reference's vocabulary
// for splitting the contraction is GlobalSplitU (src/gemm/ref/vega20_Cijk_Ailk_Bjlk_DB.yaml:69-71);
// this is the variant that needs no second kernel.
//
// A tile that spans several CTAs is finished by the CTA that holds its first slabs (the "owner":
// its run ENDS with that tile, so it reaches the tile last); the other CTAs reach their piece of
// the tile FIRST in their runs, write their partial accumulators to scratch memory and raise a
// flag.  The owner adds the partial sums in the order of the CTA indices -- a fixed order, so
// results are bit-identical from run to run -- and then applies alpha / beta and stores C.
// Waiting on a flag is bounded like every other wait of these kernels.
#pragma once

#include <stdint.h>

#include "ptx.cuh"

namespace mmbo {

struct StreamK {
  uint32_t enabled;       // host-side switch: which instantiation of the kernel is launched
  uint32_t epoch;         // what a contributor writes into its flag (the host clears the flags before the launch)
  unsigned int* flags;    // one word per CTA
  void* partials;         // one tile of accumulators per CTA, value v of thread t at [(cta * N + v) * T + t]
};

// First unit of CTA `cta` when `units` units are dealt to `grid` CTAs in contiguous runs.
__host__ __device__ __forceinline__ unsigned long long sk_first_unit(unsigned long long units, uint32_t cta,
                                                                     uint32_t grid) {
  return units * cta / grid;
}

// The work items of one CTA, in order: (tile, [kb0, kb1)).  SK = false: whole tiles with the stride of
// the grid (nothing of the stream-K machinery is compiled in); SK = true: one contiguous run of units.
template <bool SK>
struct SkWalk;

template <>
struct SkWalk<false> {
  uint32_t num_kb, tile, num_tiles;
  __device__ __forceinline__ void init(const StreamK&, uint32_t tiles, uint32_t kbs) {
    num_kb = kbs;
    tile = blockIdx.x;
    num_tiles = tiles;
  }
  __device__ __forceinline__ bool next(uint32_t* t, uint32_t* kb0, uint32_t* kb1) {
    if (tile >= num_tiles) return false;
    *t = tile;
    *kb0 = 0u;
    *kb1 = num_kb;
    tile += gridDim.x;
    return true;
  }
};

template <>
struct SkWalk<true> {
  uint32_t num_kb;
  unsigned long long u, u_end;  // units [u, u_end)
  __device__ __forceinline__ void init(const StreamK&, uint32_t tiles, uint32_t kbs) {
    num_kb = kbs;
    const unsigned long long units = (unsigned long long)tiles * kbs;
    u = sk_first_unit(units, blockIdx.x, gridDim.x);
    u_end = sk_first_unit(units, blockIdx.x + 1u, gridDim.x);
  }
  __device__ __forceinline__ bool next(uint32_t* t, uint32_t* kb0, uint32_t* kb1) {
    if (u >= u_end) return false;
    const uint32_t tt = (uint32_t)(u / num_kb);
    const uint32_t b0 = (uint32_t)(u - (unsigned long long)tt * num_kb);
    const unsigned long long left = u_end - u;
    const uint32_t b1 = left < (unsigned long long)(num_kb - b0) ? b0 + (uint32_t)left : num_kb;
    *t = tt;
    *kb0 = b0;
    *kb1 = b1;
    u += b1 - b0;
    return true;
  }
};

__device__ __forceinline__ unsigned int sk_load_flag(const unsigned int* flag) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
  return v;
}
__device__ __forceinline__ void sk_store_flag(unsigned int* flag, unsigned int v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(flag), "r"(v) : "memory");
}

// Bounded wait for a contributor's flag; false (and the fault word set) after MMBO_WAIT_LIMIT_NS.
__device__ __forceinline__ bool sk_wait_flag(const unsigned int* flag, unsigned int epoch, volatile uint32_t* abort_flag,
                                             unsigned int detail) {
#pragma unroll 1
  for (uint32_t i = 0; i < 1024u; ++i)
    if (sk_load_flag(flag) == epoch) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    if (sk_load_flag(flag) == epoch) return true;
    if ((++spins & 63u) == 0u) {
      if (*abort_flag) return false;
      if (global_timer_ns() - t0 > MMBO_WAIT_LIMIT_NS) {
        report_fault(kFaultWaitPeer, detail);
        *abort_flag = 1u;
        return false;
      }
    }
  }
}

}  // namespace mmbo
