// Tile rasterisation shared by every kernel's scheduler and by the host-side C ABI.
//
// The remap follows the reference's work-group mapping (src/gemm/ref/Kernels.cpp:209-236,
// checked on the CPU by src/gemm/ref/map.cpp:7-58): tiles are dispatched in blocks of
// `wgm` tile-columns; inside a block consecutive serial ids walk across the block's
// width first and down dimension 0 second, so that the tiles in flight at one time
// share few distinct B panels and stay resident in L2.  The last block may be
// narrower than `wgm`.
//
// All arithmetic is 32-bit (the persistent kernels evaluate this once or twice per tile
// on a single lane, where 64-bit division would cost hundreds of cycles): callers keep
// nwg0 * min(wgm, nwg1) below 2^32, which the launch code guarantees by limiting the
// tile count to 2^31.
#pragma once

#include <stdint.h>

#if defined(__CUDACC__)
#define MMBO_RASTER_HD __host__ __device__ __forceinline__
#else
#define MMBO_RASTER_HD static inline
#endif

// (wg0, wg1) of the launch grid -> (tile index along dim 0, tile index along dim 1).
MMBO_RASTER_HD void mmbo_wgm_remap(uint32_t wg0, uint32_t wg1, uint32_t nwg0, uint32_t nwg1,
                                   uint32_t wgm, uint32_t* t0, uint32_t* t1) {
  if (wgm <= 1u) {
    *t0 = wg0;
    *t1 = wg1;
    return;
  }
  const uint32_t block = wg1 / wgm;
  const uint32_t in_block = wg1 - block * wgm;
  const uint32_t serial = wg0 + in_block * nwg0;
  const uint32_t tail = nwg1 % wgm;
  const uint32_t width = (wg1 < nwg1 - tail) ? wgm : tail;
  const uint32_t q = serial / width;
  *t0 = q;
  *t1 = (serial - q * width) + block * wgm;
}

// Serial tile id of a persistent scheduler (0 .. nwg0*nwg1-1, dimension 0 fastest, the
// order in which hardware would dispatch a 2-D grid) -> tile indices.
MMBO_RASTER_HD void mmbo_tile_from_serial(uint32_t serial, uint32_t nwg0, uint32_t nwg1,
                                          uint32_t wgm, uint32_t* t0, uint32_t* t1) {
  const uint32_t wg1 = serial / nwg0;
  mmbo_wgm_remap(serial - wg1 * nwg0, wg1, nwg0, nwg1, wgm, t0, t1);
}

// ---------------------------------------------------------------------------------------------------
// The same walk without a hardware-unfriendly division: a persistent kernel evaluates the remap on one lane per
// role and tile, where each 32-bit division by a run-time value is a dependent chain of about a hundred cycles
// (four of them per tile: about 480 cycles of a 2700-cycle tile budget when the contraction is short).  The
// divisors are fixed for a launch, so the host precomputes a multiplier and a shift for each (the round-up
// method: for d >= 2, l = ceil(log2 d), mul = ceil(2^(31+l) / d), n / d = umulhi(n, mul) >> (l - 1) for every
// n < 2^31; d == 1 is flagged by mul == 0).
typedef struct MmboFastDiv {
  uint32_t mul;    // 0: the divisor is 1
  uint32_t shift;
} MmboFastDiv;

MMBO_RASTER_HD MmboFastDiv mmbo_fastdiv_make(uint32_t d) {
  MmboFastDiv f;
  f.mul = 0u;
  f.shift = 0u;
  if (d <= 1u) return f;
  uint32_t l = 0u;
  while ((1ull << l) < (unsigned long long)d) ++l;  // ceil(log2 d), 1 .. 32
  const unsigned long long two_p = 1ull << (31u + l);
  f.mul = (uint32_t)((two_p + d - 1ull) / d);
  f.shift = l - 1u;
  return f;
}

MMBO_RASTER_HD uint32_t mmbo_fastdiv(uint32_t n, MmboFastDiv f) {
#if defined(__CUDA_ARCH__)
  return f.mul ? (__umulhi(n, f.mul) >> f.shift) : n;
#else
  return f.mul ? (uint32_t)(((unsigned long long)n * f.mul) >> 32) >> f.shift : n;
#endif
}

// Everything a kernel needs to turn a serial tile id into (problem, tile row, tile column).
typedef struct MmboTileWalk {
  uint32_t nwg0, nwg1, wgm;
  uint32_t tail;        // nwg1 % wgm: width of the last, narrower block (0: none)
  uint32_t full_limit;  // nwg1 - tail: tile columns below this belong to full-width blocks
  uint32_t per_problem; // nwg0 * nwg1
  MmboFastDiv by_nwg0, by_wgm, by_tail, by_problem;
} MmboTileWalk;

MMBO_RASTER_HD MmboTileWalk mmbo_tile_walk_make(uint32_t nwg0, uint32_t nwg1, uint32_t wgm) {
  MmboTileWalk w;
  w.nwg0 = nwg0;
  w.nwg1 = nwg1;
  w.wgm = wgm;
  w.tail = wgm > 1u ? nwg1 % wgm : 0u;
  w.full_limit = nwg1 - w.tail;
  w.per_problem = nwg0 * nwg1;
  w.by_nwg0 = mmbo_fastdiv_make(nwg0);
  w.by_wgm = mmbo_fastdiv_make(wgm);
  w.by_tail = mmbo_fastdiv_make(w.tail);
  w.by_problem = mmbo_fastdiv_make(w.per_problem);
  return w;
}

// Same result as mmbo_tile_from_serial(serial, nwg0, nwg1, wgm, ...) for serial < nwg0 * nwg1 < 2^31.
MMBO_RASTER_HD void mmbo_tile_walk_locate(const MmboTileWalk w, uint32_t serial, uint32_t* t0, uint32_t* t1) {
  const uint32_t wg1 = mmbo_fastdiv(serial, w.by_nwg0);
  const uint32_t wg0 = serial - wg1 * w.nwg0;
  if (w.wgm <= 1u) {
    *t0 = wg0;
    *t1 = wg1;
    return;
  }
  const uint32_t block = mmbo_fastdiv(wg1, w.by_wgm);
  const uint32_t in_block = wg1 - block * w.wgm;
  const uint32_t ser2 = wg0 + in_block * w.nwg0;
  const int full = wg1 < w.full_limit;
  const uint32_t width = full ? w.wgm : w.tail;
  const uint32_t q = mmbo_fastdiv(ser2, full ? w.by_wgm : w.by_tail);
  *t0 = q;
  *t1 = (ser2 - q * width) + block * w.wgm;
}
