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
