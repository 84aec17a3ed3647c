/*
 * wgm_map.c -- CPU oracle for the work-group (tile) remap.  TEST INFRASTRUCTURE ONLY.
 *
 * Restates the "work-group mapping" of the reference's Tensile kernels
 * (src/gemm/ref/Kernels.cpp:209-236; the simplified power-of-two form used by the
 * hand kernels is src/gemm/assembly/naive_gemm_kernel_64_64_4_4.s:240-247):
 *
 *   serial = wg0 + (wg1 % WGM) * nwg0          position inside a block of WGM columns
 *   block  = wg1 / WGM
 *   width  = WGM, or nwg1 % WGM inside the last, partial block
 *   wg0'   = serial / width
 *   wg1'   = serial % width + block * WGM
 *
 * so that consecutively dispatched work-groups walk `width` tiles along dimension 1
 * before advancing along dimension 0, which keeps the B panels of a block resident
 * in L2.
 *
 * Pinned against the reference's golden vector src/gemm/ref/res (output of
 * src/gemm/ref/map.cpp:7-58 for nwg0 = 460, nwg1 = 64, WGM = 8): tests/test_wgm_map.py
 * checks every one of the 29 440 pairs, and, where the reference tree is present,
 * the output of map.cpp itself compiled into oracle/_ref/.
 */
#include <stdint.h>

void oracle_wgm_map(uint32_t wg0, uint32_t wg1, uint32_t nwg0, uint32_t nwg1, uint32_t wgm,
                    uint32_t *out0, uint32_t *out1) {
  uint64_t serial = (uint64_t)wg0 + (uint64_t)(wg1 % wgm) * nwg0;
  uint32_t block = wg1 / wgm;
  uint32_t rem = nwg1 % wgm;
  uint32_t width = (wg1 < nwg1 - rem) ? wgm : rem;
  *out0 = (uint32_t)(serial / width);
  *out1 = (uint32_t)(serial % width) + block * wgm;
}

/* Inverse of the map (src/gemm/ref/map.cpp:51-56 states it for full blocks only;
 * this one also inverts the partial last block). */
void oracle_wgm_unmap(uint32_t m0, uint32_t m1, uint32_t nwg0, uint32_t nwg1, uint32_t wgm,
                      uint32_t *out0, uint32_t *out1) {
  uint32_t block = m1 / wgm;
  uint32_t rem = nwg1 % wgm;
  uint32_t width = (block * wgm < nwg1 - rem) ? wgm : rem;
  uint64_t serial = (uint64_t)m0 * width + (m1 - block * wgm);
  *out0 = (uint32_t)(serial % nwg0);
  *out1 = (uint32_t)(serial / nwg0) + block * wgm;
}

/* Whole grid at once: out[2*(wg0 + wg1*nwg0) + {0,1}]. */
void oracle_wgm_map_grid(uint32_t nwg0, uint32_t nwg1, uint32_t wgm, uint32_t *out) {
  for (uint32_t j = 0; j < nwg1; ++j)
    for (uint32_t i = 0; i < nwg0; ++i)
      oracle_wgm_map(i, j, nwg0, nwg1, wgm, &out[2 * ((uint64_t)i + (uint64_t)j * nwg0)],
                     &out[2 * ((uint64_t)i + (uint64_t)j * nwg0) + 1]);
}
