// Thin inline-PTX wrappers for sm_100a: mbarrier, TMA (cp.async.bulk.tensor), tcgen05
// (tensor memory allocation, UMMA issue, commit, TMEM loads) and the fences that order
// them.  Every wait in this file is bounded: a wait that does not complete within
// MMBO_WAIT_LIMIT_NS records a code in a global status word and returns false so that
// the caller can unwind (release tensor memory, drain its copies) instead of hanging.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mmbo {

// Wall-clock bound of one barrier wait.  Real waits last microseconds to a few
// milliseconds; two seconds can only be reached by a protocol error.
#ifndef MMBO_WAIT_LIMIT_NS
#define MMBO_WAIT_LIMIT_NS 2000000000ull
#endif
// Bound used while unwinding after an error (copies already in flight land within
// microseconds).
#define MMBO_DRAIN_LIMIT_NS 20000000ull

// Device status word: 0 = ok; otherwise (code << 24) | detail of the first failure.
// Read and cleared from the host through the C ABI.
__device__ unsigned int g_mmbo_device_status = 0;

enum DeviceFault : unsigned int {
  kFaultWaitFull = 1,      // consumer gave up waiting for a TMA stage
  kFaultWaitEmpty = 2,     // producer gave up waiting for a free stage
  kFaultWaitTmemFull = 3,  // epilogue gave up waiting for an accumulator
  kFaultWaitTmemEmpty = 4, // MMA issuer gave up waiting for a drained accumulator
  kFaultWaitCLoad = 5,     // epilogue gave up waiting for its C tile
  kFaultTmemAlloc = 6,     // tensor memory allocation returned an unexpected address
  kFaultWaitPeer = 7,      // CTA pair handshake timed out
};

__device__ __forceinline__ void report_fault(unsigned int code, unsigned int detail) {
  atomicCAS(&g_mmbo_device_status, 0u, (code << 24) | (detail & 0xffffffu));
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------- mbarrier ----------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Arrive on a barrier of another CTA of the cluster (address from mapa).  The arrive carries the default
// CTA-scope release: what it hands over here is tensor memory, whose reads are ordered by tcgen05.wait::ld and
// tcgen05.fence::before_thread_sync, not generic memory.  (A cluster-scope release makes the thread wait for all
// of its memory traffic in flight -- measured: ~1000 cycles per arrive, 1500-2900 with TMA stores outstanding,
// which put every tile's release behind the previous tile's stores.)  -DMMBO_RELEASE_CLUSTER=1 restores it.
#ifndef MMBO_RELEASE_CLUSTER
#define MMBO_RELEASE_CLUSTER 0
#endif
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
#if MMBO_RELEASE_CLUSTER
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
#else
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
#endif
}

__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t cta_rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(cta_rank));
  return out;
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  `abort_flag` is a word in shared memory that any role sets when it
// gives up; once set, every other wait returns false quickly.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          unsigned int fault_code, unsigned int detail,
                                          uint64_t limit_ns = MMBO_WAIT_LIMIT_NS) {
  // Fast path: poll without touching the global timer (reading it costs far more than
  // a poll, and almost every wait ends within a few polls).
#pragma unroll 1
  for (uint32_t i = 0; i < 1024u; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  // A wait that has lasted this long is a long one (a whole main loop, a busy copy engine): back off
  // between polls so that the waiting thread stops competing for issue slots and power.
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    __nanosleep(128);
    if ((++spins & 63u) == 0u) {
      if (*abort_flag) return false;
      if (global_timer_ns() - t0 > limit_ns) {
        report_fault(fault_code, detail);
        *abort_flag = 1u;
        return false;
      }
    }
  }
}

// The same for a whole (converged) warp: lane 0 polls, the other lanes rest at the shuffle; once the
// phase has completed every lane observes it itself (one poll that succeeds at once), which gives each
// lane the ordering a wait of its own would have given.  The result is warp-uniform.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                               unsigned int fault_code, unsigned int detail) {
  // Fast path: the phase has usually completed already when an epilogue warp gets here (it is the slower
  // side with short contractions): all lanes poll once, and agree.
  if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) return true;
  uint32_t ok = 1u;
  if ((threadIdx.x & 31u) == 0u) ok = mbar_wait(bar, parity, abort_flag, fault_code, detail) ? 1u : 0u;
  ok = __shfl_sync(0xffffffffu, ok, 0);
  if (ok) {
#pragma unroll 1
    for (uint32_t i = 0; i < 64u && !mbar_try_wait(bar, parity); ++i) {
    }
  }
  return ok != 0u;
}

// ---------------------------------------------------------------- packed fp32 ---------
// Two fp32 values in one 64-bit register; sm_100 multiplies and fuses them in one instruction
// (each half is rounded exactly as the scalar instruction would round it).
__device__ __forceinline__ uint64_t pack_f32x2(uint32_t lo, uint32_t hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ uint64_t mul_f32x2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
// {lo, hi} fp16 pair (lo in the low 16 bits, as stored in memory) <-> packed fp32 pair
// (Widening with the mixed-precision add.rn.f32.f16 x, -0.0 is exact too -- checked on all 65536 halves -- but it
// issues at the same rate as cvt.f32.f16, one per ~9 cycles and scheduler, so the conversion stays.)
__device__ __forceinline__ uint64_t half2_to_f32x2(uint32_t h2) {
  uint32_t lo, hi;
  asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\tcvt.f32.f16 %0, l;\n\tcvt.f32.f16 %1, h;\n\t}"
      : "=r"(lo), "=r"(hi)
      : "r"(h2));
  return pack_f32x2(lo, hi);
}
__device__ __forceinline__ uint32_t f32x2_to_half2(uint64_t v) {
  uint32_t lo, hi, r;
  asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(v));
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "r"(hi), "r"(lo));  // first source -> upper half
  return r;
}

// ---------------------------------------------------------------- fences -------------
// Programmatic dependent launch (no-ops in a grid launched without the attribute): let the next kernel of the
// stream start its set-up; wait until the previous kernel has completed and its writes are visible.
__device__ __forceinline__ void griddep_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void griddep_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------- TMA ----------------
// 2-D tiled load, completion on an mbarrier of this CTA.  c0 is the coordinate along
// the contiguous dimension and must keep c0 * element size a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int32_t c0, int32_t c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

// Same, issued by either CTA of a pair: the barrier address may name the peer CTA's
// barrier (shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map,
                                                 uint32_t cluster_bar, int32_t c0, int32_t c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(c0), "r"(c1)
      : "memory");
}

// 3-D forms: the third coordinate is the problem index of a strided batch (the tensor map's
// outermost dimension, one problem per index); it has no alignment rule.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int32_t c0, int32_t c1, int32_t c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map,
                                                 uint32_t cluster_bar, int32_t c0, int32_t c1, int32_t c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_l2_3d(const CUtensorMap* map, int32_t c0, int32_t c1, int32_t c2) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global [%0, {%1, %2, %3}];" ::"l"(map), "r"(c0), "r"(c1),
               "r"(c2)
               : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int32_t c0, int32_t c1,
                                             int32_t c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}

// Asks L2 to fetch a tile ahead of the load that will need it (no shared memory involved).
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap* map, int32_t c0, int32_t c1) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];" ::"l"(map), "r"(c0), "r"(c1)
               : "memory");
}

// C is written once per launch: its lines are marked to leave L2 first, so that they do not push out operand panels
// that other CTAs are about to read again (8192 x 8192 x 256: 38.2 -> 37.6 us; long contractions unchanged; an
// evict-last hint on the operand loads made no measurable difference and is not used).  -DMMBO_L2_HINTS=0: no hint.
#ifndef MMBO_L2_HINTS
#define MMBO_L2_HINTS 1
#endif
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int32_t c0,
                                             int32_t c1) {
#if MMBO_L2_HINTS & 1
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%2, %3}], [%1], %4;"
               ::"l"(map), "r"(src), "r"(c0), "r"(c1), "l"(l2_policy_evict_first())
               : "memory");
#else
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(src), "r"(c0), "r"(c1)
               : "memory");
#endif
}

// Single problems keep 2-D tensor maps and the 2-D instruction forms; a strided batch uses 3-D maps.
// `batched` is uniform over the grid, so the branch costs nothing.
__device__ __forceinline__ void tma_load_tile(bool batched, uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                              int32_t c0, int32_t c1, int32_t c2) {
  if (batched) tma_load_3d(dst, map, bar, c0, c1, c2);
  else tma_load_2d(dst, map, bar, c0, c1);
}
__device__ __forceinline__ void tma_load_tile_pair(bool batched, uint32_t dst, const CUtensorMap* map,
                                                   uint32_t cluster_bar, int32_t c0, int32_t c1, int32_t c2) {
  if (batched) tma_load_3d_pair(dst, map, cluster_bar, c0, c1, c2);
  else tma_load_2d_pair(dst, map, cluster_bar, c0, c1);
}
__device__ __forceinline__ void tma_prefetch_l2_tile(bool batched, const CUtensorMap* map, int32_t c0, int32_t c1,
                                                     int32_t c2) {
  if (batched) tma_prefetch_l2_3d(map, c0, c1, c2);
  else tma_prefetch_l2_2d(map, c0, c1);
}
__device__ __forceinline__ void tma_store_tile(bool batched, const CUtensorMap* map, uint32_t src, int32_t c0,
                                               int32_t c1, int32_t c2) {
  if (batched) tma_store_3d(map, src, c0, c1, c2);
  else tma_store_2d(map, src, c0, c1);
}

// 16-byte store to a multicast address (an address range that NVSwitch maps onto the same offset
// of a buffer in several GPUs): every GPU bound to the range receives the data.  A store only;
// nothing is ever loaded through such an address here.
__device__ __forceinline__ void multimem_st_v4(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

template <int N>
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---------------------------------------------------------------- tensor memory ------
template <int CTA_GROUP>
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols) {
  if constexpr (CTA_GROUP == 1)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result),
                 "r"(ncols)
                 : "memory");
  else
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result),
                 "r"(ncols)
                 : "memory");
}

template <int CTA_GROUP>
__device__ __forceinline__ void tmem_relinquish() {
  if constexpr (CTA_GROUP == 1)
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  else
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

template <int CTA_GROUP>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  if constexpr (CTA_GROUP == 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
  else
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc]; issued by one thread.
template <int CTA_GROUP, bool TF32>
__device__ __forceinline__ void umma_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                        uint32_t idesc, uint32_t accumulate) {
  if constexpr (CTA_GROUP == 1 && !TF32)
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
  else if constexpr (CTA_GROUP == 2 && !TF32)
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
  else if constexpr (CTA_GROUP == 1 && TF32)
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
  else
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// CTA-pair fp16 UMMA that keeps its A operand in the tensor core's collector buffer (FILL) for the next
// UMMA, which takes it from there instead of reading shared memory again (LASTUSE) -- for consecutive UMMAs
// on the same A descriptor (a tile taller than one UMMA: same op(B) operand, next piece of op(A)).
template <bool LASTUSE>
__device__ __forceinline__ void umma_ss_pair_f16_collect_a(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                                          uint32_t idesc, uint32_t accumulate) {
  if constexpr (!LASTUSE)
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16.collector::a::fill [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
  else
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16.collector::a::lastuse [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Arrive on an mbarrier of this CTA once every UMMA issued so far by this thread has
// finished (implies tcgen05.fence::before_thread_sync).
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// CTA-pair form: arrives on the barrier at the same offset in every CTA named by
// cta_mask (bit r = CTA rank r of the cluster).  This is a barrier signal, not a data
// copy.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"(cta_mask)
      : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp receives lane
// (base lane + t), columns [col, col + 32).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------- descriptors --------
// Shared-memory matrix descriptor for a 128-byte-swizzled operand tile whose base is
// 1024-byte aligned.  Offsets are in bytes; the fields hold them divided by 16.
//   K-major  (contraction index contiguous): rows of 128 bytes, groups of 8 rows are
//            `sbo` bytes apart; `lbo` is not used by the hardware for swizzled layouts.
//   MN-major (row/column index contiguous): spans of 128 bytes along MN x 8 k-rows form
//            a 1024-byte atom; atoms are `sbo` bytes apart along K and `lbo` bytes apart
//            along MN.
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes,
                                                         uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fffu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fffu) << 32;
  d |= static_cast<uint64_t>(1) << 46;  // descriptor version of this architecture
  d |= static_cast<uint64_t>(2) << 61;  // 128-byte swizzle
  return d;
}

// Instruction descriptor for kind::f16 / kind::tf32 with fp32 accumulation.
//   ab_format: 0 = f16, 1 = bf16, 2 = tf32;  *_mn_major: 1 when the operand's smem tile
//   has its M (or N) index contiguous instead of K.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t ab_format, uint32_t a_mn_major,
                                                  uint32_t b_mn_major, uint32_t mma_m,
                                                  uint32_t mma_n) {
  return (1u << 4)                 // D format: f32
         | (ab_format << 7)        // A format
         | (ab_format << 10)       // B format
         | (a_mn_major << 15)      // A major-ness
         | (b_mn_major << 16)      // B major-ness
         | ((mma_n >> 3) << 17)    // N / 8
         | ((mma_m >> 4) << 24);   // M / 16
}

}  // namespace mmbo
