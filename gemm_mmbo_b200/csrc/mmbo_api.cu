// C ABI of libmmbo_gemm.so: argument validation, kernel table, kernel selection, tensor
// map construction and launches.  Counterpart of the reference's launch surface
// (src/gemm/gemm.h:4-97 packs arguments and picks a table row; src/gemm/driver.h:15-61
// loads a code object and launches it).  Unlike the reference nothing is loaded per
// call: every kernel is linked into this library.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <type_traits>
#include <stdint.h>
#include <stdio.h>

#include <mutex>
#include <stdlib.h>
#include <string.h>

#include "../../include/mmbo_gemm.h"
#include "dgemm_dmma.cuh"
#include "dgemm_dmma_ws.cuh"
#include "sgemm_ffma_ws.cuh"
#include "dgemm_fma.cuh"
#include "hgemm_tcgen05.cuh"
#include "nccl_dl.h"
#include "ref_kernels.cuh"
#include "sgemm_ffma.cuh"
#include "sgemm_tf32x3.cuh"

namespace mmbo {

// ------------------------------------------------------------------ kernel table -----
struct KernelRow {
  const char* name;
  int mt0, mt1, threads, depth_u, stages, cta_group, wgm, tensor;
};

// fp32 rows.  Names follow the reference's scheme (src/gemm/constants.h:20-33):
// MT<tile m>x<tile n>x<DepthU>_TT<thread tile>_WG<threads>.
static const KernelRow kF32Rows[] = {
    {"sgemm_simple_MT032x008x01_TT01_01_WG256", 32, 8, 256, 1, 1, 1, 1, 0},
    {"sgemm_ffma_MT128x128x16_TT08_08_WG256_WGM08", 128, 128, 256, 16, 2, 1, 8, 0},
    {"sgemm_ffma_MT064x064x16_TT04_04_WG256_WGM08", 64, 64, 256, 16, 2, 1, 8, 0},
    {"sgemm_tf32x3_tcgen05_MT128x256x32_S4_CG2_WG192_WGM08", 128, 256, 192, 32, 4, 2, 8, 1},
    {"sgemm_tf32x3_tcgen05_MT128x128x32_S3_CG1_WG192_WGM08", 128, 128, 192, 32, 3, 1, 8, 1},
    {"sgemm_tf32x3_tcgen05_MT256x256x32_S3_CG2_WG384_WGM08", 256, 256, 384, 32, 3, 2, 8, 1},
    {"sgemm_ffma_ws_MT128x128x16_S4_TT08_08_WG384_WGM08", 128, 128, 384, 16, 4, 1, 8, 0},
};
// fp16 rows: MT<tile m>x<tile n>x<DepthU>_S<stages>_CG<cta group>.
static const KernelRow kF16Rows[] = {
    {"hgemm_simple_MT032x008x01_TT01_01_WG256", 32, 8, 256, 1, 1, 1, 1, 0},
    {"hgemm_tcgen05_MT256x128x64_S4_CG1_WG192_WGM08", 256, 128, 192, 64, 4, 1, 8, 1},
    {"hgemm_tcgen05_MT128x128x64_S6_CG1_WG192_WGM08", 128, 128, 192, 64, 6, 1, 8, 1},
    {"hgemm_tcgen05_MT256x256x64_S6_CG2_WG192_WGM08", 256, 256, 192, 64, 6, 2, 8, 1},
    {"hgemm_tcgen05_MT256x256x64_S3_CG2_WG320_WGM08", 256, 256, 320, 64, 3, 2, 8, 1},
    {"hgemm_tcgen05_MT256x256x64_S5_CG2_WG320_WGM08", 256, 256, 320, 64, 5, 2, 8, 1},
    {"hgemm_tcgen05_MT512x256x64_S4_CG2_WG192_WGM08", 512, 256, 192, 64, 4, 2, 8, 1},
    {"hgemm_tcgen05_MT512x256x64_S4_CG2_WG320_WGM08", 512, 256, 320, 64, 4, 2, 8, 1},
};
// fp64 rows (the reference's own dtype).
static const KernelRow kF64Rows[] = {
    {"dgemm_simple_MT032x008x01_TT01_01_WG256", 32, 8, 256, 1, 1, 1, 1, 0},
    {"dgemm_fma_MT064x064x16_TT04_04_WG256_WGM08", 64, 64, 256, 16, 2, 1, 8, 0},
    {"dgemm_dmma_MT128x064x08_WT32_32_WG256_WGM08", 128, 64, 256, 8, 2, 1, 8, 1},
    {"dgemm_dmma_ws_MT128x064x16_S4_WT64_32_WG256_WGM08", 128, 64, 256, 16, 4, 1, 8, 1},
    {"dgemm_dmma_ws_MT064x064x16_S4_WT32_32_WG256_WGM08", 64, 64, 256, 16, 4, 1, 8, 1},
};
constexpr int kNumF64 = sizeof(kF64Rows) / sizeof(KernelRow);
constexpr int kNumF32 = sizeof(kF32Rows) / sizeof(KernelRow);
constexpr int kNumF16 = sizeof(kF16Rows) / sizeof(KernelRow);

static const KernelRow* rows_of(int dtype, int* count) {
  if (dtype == MMBO_DTYPE_F32) {
    *count = kNumF32;
    return kF32Rows;
  }
  if (dtype == MMBO_DTYPE_F16) {
    *count = kNumF16;
    return kF16Rows;
  }
  if (dtype == MMBO_DTYPE_F64) {
    *count = kNumF64;
    return kF64Rows;
  }
  *count = 0;
  return nullptr;
}

// One lock for the library's host-side state (per-device caches of attributes, scratch
// buffers, staging pipes, the tuning table, the trace buffer).  Entry points that launch
// take it for the duration of the call, so concurrent callers are serialised on the host
// only; the work they queue still overlaps on the GPU.
static std::recursive_mutex g_api_mutex;
#define MMBO_API_LOCK() std::lock_guard<std::recursive_mutex> mmbo_api_lock_(g_api_mutex)

// ------------------------------------------------------------------ device info ------
constexpr int kMaxDevices = 64;
static int g_sm_count[kMaxDevices];

static int current_device() {
  int dev = 0;
  cudaGetDevice(&dev);
  return dev;
}

static int sm_count() {
  const int dev = current_device();
  if (dev < 0 || dev >= kMaxDevices) return 148;
  if (g_sm_count[dev] == 0) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) {
      cudaGetLastError();
      v = 148;
    }
    g_sm_count[dev] = v;
  }
  return g_sm_count[dev];
}

static uint32_t env_u32(const char* name, uint32_t fallback) {
  const char* s = getenv(name);
  if (!s || !*s) return fallback;
  return (uint32_t)strtoul(s, nullptr, 10);
}

// Switches for experiments and diagnosis.  The environment is read ONCE, when the first
// call needs a setting; afterwards only mmbo_set_option changes them, so that a launch
// costs no getenv scan and a production process cannot be flipped into a diagnostic
// mode by an environment change after start-up.
struct Settings {
  uint32_t diag;           // MMBO_DIAG: diagnostic kernels, results wrong by design (bit 0 no C store, bit 1 no drain)
  uint32_t wgm;            // MMBO_WGM: work-group-mapping width for every kernel; 0 = the table row's
  uint32_t tf32_chunk;     // MMBO_TF32_CHUNK: stages per tensor-memory accumulation chain of the 3xTF32 kernels
  uint32_t f32_exact;      // MMBO_F32_EXACT: automatic fp32 selection stays on the CUDA-core kernels
  uint32_t dgemm_stage_c;  // MMBO_DGEMM_STAGE_C: 64-row fp64 tiles stage the old C through shared memory
  uint32_t split_k;        // MMBO_SPLIT_K: 0 = automatic, 1 = never split, n > 1 = force n slices where a kernel can
  uint32_t pdl;            // MMBO_PDL: the persistent tcgen05 kernels are launched with programmatic stream serialization
                           // (their set-up overlaps the end of the previous kernel of the stream); 0 switches it off
};
static Settings load_settings() {
  Settings s;
  s.diag = env_u32("MMBO_DIAG", 0);
  s.wgm = env_u32("MMBO_WGM", 0);
  s.tf32_chunk = env_u32("MMBO_TF32_CHUNK", 4);
  if (s.tf32_chunk == 0) s.tf32_chunk = 1;
  s.f32_exact = env_u32("MMBO_F32_EXACT", 0);
  s.dgemm_stage_c = env_u32("MMBO_DGEMM_STAGE_C", 1);
  s.split_k = env_u32("MMBO_SPLIT_K", 0);
  s.pdl = env_u32("MMBO_PDL", 1);
  return s;
}
static Settings& settings() {
  static Settings s = load_settings();
  return s;
}
static uint32_t wgm_of(const KernelRow& row) { return settings().wgm ? settings().wgm : (uint32_t)row.wgm; }

// Kernel launches queued by this library since it was loaded (every <<<>>> and
// cudaLaunchKernelEx of a GEMM, split or scale kernel; not the operand generator).
static unsigned long long g_launch_count = 0;
#define MMBO_COUNT_LAUNCH() (++g_launch_count)

// ------------------------------------------------------------------ validation -------
struct GemmArgs {
  int transA, transB;
  size_t m, n, k;
  const void *A, *B;
  void* C;
  size_t lda, ldb, ldc;
  float alpha, beta;
  // fp16 tensor-core kernels only: further copies of the C window (peer GPUs) the epilogue stores to
  void* const* peers = nullptr;
  int npeers = 0;
  // ... or one multicast address of the same window (NVSwitch replicates each store to every GPU bound to it)
  void* c_multicast = nullptr;
  // strided batch: `batch` problems whose operands are sA / sB / sC elements apart
  size_t batch = 1, sA = 0, sB = 0, sC = 0;
};

static int validate(const GemmArgs& g, const float* alpha, const float* beta) {
  if ((g.transA != 0 && g.transA != 1) || (g.transB != 0 && g.transB != 1)) return MMBO_ERR_BAD_TRANS;
  const size_t lim = 0x7fffffffull;
  if (g.m > lim || g.n > lim || g.k > lim) return MMBO_ERR_BAD_DIM;
  if (!alpha || !beta) return MMBO_ERR_NULL_POINTER;
  if (g.m == 0 || g.n == 0) return MMBO_OK;
  if (!g.C) return MMBO_ERR_NULL_POINTER;
  if (g.ldc < g.m || g.ldc > lim) return MMBO_ERR_BAD_LDC;
  if (g.k != 0) {
    if (!g.A || !g.B) return MMBO_ERR_NULL_POINTER;
    if (g.lda < (g.transA ? g.k : g.m) || g.lda > lim) return MMBO_ERR_BAD_LDA;
    if (g.ldb < (g.transB ? g.n : g.k) || g.ldb > lim) return MMBO_ERR_BAD_LDB;
  }
  return MMBO_OK;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ------------------------------------------------------------------ TMA maps ---------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;
static bool g_encode_tried = false;

static EncodeTiledFn encode_fn() {
  if (!g_encode_tried) {
    g_encode_tried = true;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    else
      cudaGetLastError();
  }
  return g_encode;
}

// Map over a column-major array (or a strided batch of them): dimension 0 (contiguous) has
// `inner` elements, dimension 1 has `outer` elements `ld` elements apart and, for a batch, dimension 2
// has `nbatch` problems `batch_stride` elements apart.  128-byte swizzle by default; out-of-range elements read as zero.
static int make_map(CUtensorMap* map, CUtensorMapDataType dt, size_t elem_bytes, const void* base,
                    size_t inner, size_t outer, size_t ld, uint32_t box_inner, uint32_t box_outer,
                    CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B, size_t nbatch = 1,
                    size_t batch_stride = 0) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return MMBO_ERR_NO_DRIVER_ENTRY;
  cuuint64_t dims[3] = {inner, outer, nbatch};
  cuuint64_t strides[2] = {ld * elem_bytes, batch_stride * elem_bytes};
  cuuint32_t box[3] = {box_inner, box_outer, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  // a single problem is a 2-D map (the kernels then use the 2-D instruction forms)
  CUresult r = enc(map, dt, nbatch > 1 ? 3 : 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? MMBO_OK : MMBO_ERR_TENSOR_MAP;
}

// Plain 2-D map (the peer copies of C, which the epilogue addresses with two coordinates).
static int make_map_2d(CUtensorMap* map, CUtensorMapDataType dt, size_t elem_bytes, const void* base,
                       size_t inner, size_t outer, size_t ld, uint32_t box_inner, uint32_t box_outer,
                       CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return MMBO_ERR_NO_DRIVER_ENTRY;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * elem_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? MMBO_OK : MMBO_ERR_TENSOR_MAP;
}

// A batch stride TMA can take: a multiple of 16 bytes below 2^40 (a single problem has none).
static bool batch_stride_ok(size_t batch, size_t stride_elems, size_t elem_bytes) {
  if (batch <= 1) return true;
  const unsigned long long b = (unsigned long long)stride_elems * elem_bytes;
  return stride_elems != 0 && b % 16 == 0 && b < (1ull << 40);
}

// Self-test of the bounded-wait machinery: one thread waits on a barrier that nothing
// will ever complete, with a short limit; it must give up, record its fault code and
// return, leaving the context usable.
__global__ void bounded_wait_selftest_kernel(unsigned long long limit_ns) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0u;
    mbar_init(smem_u32(&bar), 1);
    fence_mbar_init();
    mbar_wait(smem_u32(&bar), 0u, &abort_flag, kFaultWaitPeer, 0x5e1f, limit_ns);
  }
}

// Device buffer for the optional event trace of the tcgen05 kernels (see trace_stamp).
static unsigned long long* g_trace_buffer = nullptr;
constexpr size_t kTraceWords = 64 * 16;

// ------------------------------------------------------------------ scratch memory --
// One scratch buffer per device, used by the kernels that repack operands (the 3xTF32
// SGEMM, fp16 operands TMA cannot address, split-K partial sums).  Either the caller lends
// one (mmbo_set_workspace) or the library grows its own on demand.  Calls that use it are
// ordered on the GPU by the library itself: every user records an event behind its last
// kernel, and the next user on a DIFFERENT stream first makes its stream wait for that
// event, so that two streams never work in the buffer at the same time (the reference's
// kernels use no scratch, so a caller coming from it has no reason to expect a hazard).
struct Workspace {
  void* ptr;
  size_t bytes;
  bool user;
  cudaEvent_t last_use;      // recorded behind the last kernel that used the buffer
  cudaStream_t last_stream;  // stream of that kernel
  bool used;
};
static Workspace g_ws[kMaxDevices];

static int ensure_workspace(size_t bytes, void** out) {
  const int dev = current_device();
  if (dev < 0 || dev >= kMaxDevices) return MMBO_ERR_TOO_LARGE;
  Workspace& w = g_ws[dev];
  if (w.bytes < bytes) {
    if (w.user) return MMBO_ERR_WORKSPACE;
    if (w.ptr) {
      cudaError_t e = cudaFree(w.ptr);  // waits for the kernels still using it
      w.ptr = nullptr;
      w.bytes = 0;
      w.used = false;
      if (e != cudaSuccess) return (int)e;
    }
    cudaError_t e = cudaMalloc(&w.ptr, bytes);
    if (e != cudaSuccess) {
      w.ptr = nullptr;
      return (int)e;
    }
    w.bytes = bytes;
  }
  *out = w.ptr;
  return MMBO_OK;
}

// Called before the first kernel of a call that uses the scratch buffer ...
static int workspace_acquire(cudaStream_t st) {
  const int dev = current_device();
  if (dev < 0 || dev >= kMaxDevices) return MMBO_ERR_TOO_LARGE;
  Workspace& w = g_ws[dev];
  if (w.used && w.last_stream != st) {
    cudaError_t e = cudaStreamWaitEvent(st, w.last_use, 0);
    if (e != cudaSuccess) return (int)e;
  }
  return MMBO_OK;
}
// ... and behind its last one.
static int workspace_release(cudaStream_t st) {
  const int dev = current_device();
  if (dev < 0 || dev >= kMaxDevices) return MMBO_ERR_TOO_LARGE;
  Workspace& w = g_ws[dev];
  if (!w.last_use) {
    cudaError_t e = cudaEventCreateWithFlags(&w.last_use, cudaEventDisableTiming);
    if (e != cudaSuccess) return (int)e;
  }
  cudaError_t e = cudaEventRecord(w.last_use, st);
  if (e != cudaSuccess) return (int)e;
  w.last_stream = st;
  w.used = true;
  return MMBO_OK;
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Stream-K (stream_k.cuh) for the persistent producer / consumer kernels: decided per call.  `slots` = CTAs
// resident at once; a unit is one k-slab of one tile.  Splitting pays when whole-tile rounds leave the last
// round part empty; each CTA then writes or reads at most one tile of partial sums (about `overhead_units`
// slabs' worth of time).  split_k = 1 switches it off, > 1 forces it wherever the problem has enough slabs.
struct SkPlan {
  bool on;
  unsigned grid;
  size_t flag_bytes, total_bytes;
};
// Split mode the tuning table holds for the problem of the call in progress (0: none); set by the table
// lookup of automatic selection, consulted when the option itself says "automatic".
static uint32_t g_split_from_table = 0;

static SkPlan plan_stream_k(size_t tiles, size_t num_kb, size_t slots, size_t partial_bytes, int warps, size_t batch) {
  SkPlan pl{false, 0, 0, 0};
  const uint32_t mode = settings().split_k ? settings().split_k : g_split_from_table;
  const unsigned long long units = (unsigned long long)tiles * num_kb;
  if (mode == 1 || batch != 1 || tiles == 0 || num_kb < 8 || units >= (1ull << 40)) return pl;
  size_t grid = slots;
  if (units / 8 < grid) grid = (size_t)(units / 8);  // at least 8 slabs per CTA
  if (grid < 2) return pl;
  if (mode == 0) {
    const double overhead_units = 6.0;
    const double dp = (double)((tiles + slots - 1) / slots) * (double)num_kb;
    const double sk = (double)units / (double)grid + overhead_units;
    if (!(dp > 1.04 * sk)) return pl;
  }
  pl.on = true;
  pl.grid = (unsigned)grid;
  pl.flag_bytes = align_up(grid * (size_t)warps * 4, 1024);
  pl.total_bytes = pl.flag_bytes + grid * partial_bytes;
  return pl;
}
// Scratch of a stream-K launch: cleared flags first, one tile of partial sums per CTA behind them.
static int prepare_stream_k(const SkPlan& pl, cudaStream_t st, StreamK* sk) {
  sk->enabled = 0; sk->epoch = 1; sk->flags = nullptr; sk->partials = nullptr;
  if (!pl.on) return MMBO_OK;
  void* scratch = nullptr;
  int rc = ensure_workspace(pl.total_bytes, &scratch);
  if (rc) return rc;
  if ((rc = workspace_acquire(st))) return rc;
  cudaError_t e = cudaMemsetAsync(scratch, 0, pl.flag_bytes, st);
  if (e != cudaSuccess) return (int)e;
  sk->enabled = 1;
  sk->flags = static_cast<unsigned int*>(scratch);
  sk->partials = static_cast<char*>(scratch) + pl.flag_bytes;
  return MMBO_OK;
}

// ------------------------------------------------------------------ launches ---------
template <typename T>
static int launch_simple(const GemmArgs& g, cudaStream_t st) {
  const size_t gx = (g.m + 31) / 32, gy = (g.n + 7) / 8;
  if (gy > 65535 || gx > 0x7fffffffull || g.batch > 65535) return MMBO_ERR_TOO_LARGE;
  dim3 grid((unsigned)gx, (unsigned)gy, (unsigned)g.batch), block(32, 8);
  gemm_simple_kernel<T><<<grid, block, 0, st>>>(g.transA, g.transB, g.m, g.n, g.k, g.alpha,
                                                static_cast<const T*>(g.A), g.lda,
                                                static_cast<const T*>(g.B), g.ldb, g.beta,
                                                static_cast<T*>(g.C), g.ldc, g.sA, g.sB, g.sC);
  MMBO_COUNT_LAUNCH();
  return (int)cudaGetLastError();
}

template <typename T>
static int launch_scale(const GemmArgs& g, cudaStream_t st) {
  const size_t gx = (g.m + 31) / 32, gy = (g.n + 7) / 8;
  if (gy > 65535 || gx > 0x7fffffffull || g.batch > 65535) return MMBO_ERR_TOO_LARGE;
  dim3 grid((unsigned)gx, (unsigned)gy, (unsigned)g.batch), block(32, 8);
  scale_c_kernel<T><<<grid, block, 0, st>>>(g.m, g.n, g.beta, static_cast<T*>(g.C), g.ldc, g.sC);
  MMBO_COUNT_LAUNCH();
  return (int)cudaGetLastError();
}

// FFMA kernel with a producer warpgroup: an operand goes through TMA when its tile rows are
// contiguous in memory, its base 16-byte aligned and its leading dimension a multiple of 4.
static int launch_sgemm_ffma_ws(const GemmArgs& g, uint32_t wgm, cudaStream_t st) {
  SgemmParams p;
  p.m = (uint32_t)g.m; p.n = (uint32_t)g.n; p.k = (uint32_t)g.k;
  p.lda = (uint32_t)g.lda; p.ldb = (uint32_t)g.ldb; p.ldc = (uint32_t)g.ldc;
  p.alpha = g.alpha; p.beta = g.beta; p.wgm = wgm;
  p.batch_a = p.batch_b = p.batch_c = 0;
  p.vec_a = p.vec_b = 0;
  p.vec_c = aligned16(g.C) && g.ldc % 4 == 0;
  SgemmWsFlags f;
  f.tma_a = !g.transA && aligned16(g.A) && g.lda % 4 == 0;
  f.tma_b = g.transB && aligned16(g.B) && g.ldb % 4 == 0;
  CUtensorMap ta, tb;
  memset(&ta, 0, sizeof(ta));
  memset(&tb, 0, sizeof(tb));
  if (f.tma_a) {
    const int rc = make_map_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, g.A, g.m, g.k, g.lda, kFwBM + kFwPad, kFwBK,
                               CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
  }
  if (f.tma_b) {
    const int rc = make_map_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, g.B, g.n, g.k, g.ldb, kFwBN + kFwPad, kFwBK,
                               CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
  }
  const size_t tiles = ((g.m + kFwBM - 1) / kFwBM) * ((g.n + kFwBN - 1) / kFwBN);
  if (tiles > 0x7fffffffull) return MMBO_ERR_TOO_LARGE;
  // Eight CTAs per SM in the grid, two resident: as CTAs finish their few tiles the hardware starts the
  // next ones, which balances the end of the launch (4096^3: 61.1 TFLOP/s against 52.3 with 2 per SM).
  unsigned grid = (unsigned)std::min(tiles, (size_t)8 * (size_t)sm_count());
  // Few tiles (fewer than two per resident CTA): stream-K over the two resident CTAs per SM instead (all of
  // them run at once, which the flag hand-over between CTAs relies on): 1024^3 22.9 -> 33.0 TFLOP/s, 2048^3
  // 49.3 -> 52.8.  With more tiles the oversubscribed grid already balances the end of the launch and the
  // split only costs (4096^3 NN / NT / TN: 58.3 / 61.1 / 54.9 without, 55.6 / 59.3 / 52.4 with).
  SkPlan plan{false, 0, 0, 0};
  if (tiles < (size_t)4 * (size_t)sm_count())
    plan = plan_stream_k(tiles, (g.k + kFwBK - 1) / kFwBK, (size_t)2 * (size_t)sm_count(), (size_t)kFwBM * kFwBN * 4,
                         kFwConsumerWarps, g.batch);
  StreamK sk;
  {
    const int rc = prepare_stream_k(plan, st, &sk);
    // scratch that cannot be had (a lent buffer that is too small) is no error: whole tiles then
    if (rc == MMBO_OK && plan.on) grid = plan.grid;
    else sk.enabled = 0;
  }
  const float* A = static_cast<const float*>(g.A);
  const float* B = static_cast<const float*>(g.B);
  float* C = static_cast<float*>(g.C);
  auto launch = [&](auto kernel) -> int {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFwSmemBytes);
    if (e != cudaSuccess) return (int)e;
    kernel<<<grid, kFwThreads, kFwSmemBytes, st>>>(ta, tb, A, B, C, p, f, sk);
    MMBO_COUNT_LAUNCH();
    int rc = (int)cudaGetLastError();
    if (sk.enabled) {
      const int rc2 = workspace_release(st);
      if (!rc) rc = rc2;
    }
    return rc;
  };
  if (sk.enabled) {
    if (!g.transA && !g.transB) return launch(sgemm_ffma_ws_kernel<false, false, true>);
    if (!g.transA && g.transB) return launch(sgemm_ffma_ws_kernel<false, true, true>);
    if (g.transA && !g.transB) return launch(sgemm_ffma_ws_kernel<true, false, true>);
    return launch(sgemm_ffma_ws_kernel<true, true, true>);
  }
  if (!g.transA && !g.transB) return launch(sgemm_ffma_ws_kernel<false, false>);
  if (!g.transA && g.transB) return launch(sgemm_ffma_ws_kernel<false, true>);
  if (g.transA && !g.transB) return launch(sgemm_ffma_ws_kernel<true, false>);
  return launch(sgemm_ffma_ws_kernel<true, true>);
}

template <int BM, int BN, int TTM, int TTN>
static int launch_sgemm_ffma(const GemmArgs& g, uint32_t wgm, cudaStream_t st) {
  constexpr int BK = 16;
  SgemmParams p;
  p.m = (uint32_t)g.m; p.n = (uint32_t)g.n; p.k = (uint32_t)g.k;
  p.lda = (uint32_t)g.lda; p.ldb = (uint32_t)g.ldb; p.ldc = (uint32_t)g.ldc;
  p.alpha = g.alpha; p.beta = g.beta; p.wgm = wgm;
  p.batch_a = g.sA; p.batch_b = g.sB; p.batch_c = g.sC;
  // 128-bit accesses: base and pitch 16-byte aligned, and the contiguous extent a
  // multiple of 4 so that no vector straddles the matrix edge (every problem of a batch).
  const bool batched = g.batch > 1;
  const size_t a_contig = g.transA ? g.k : g.m, b_contig = g.transB ? g.n : g.k;
  p.vec_a = aligned16(g.A) && g.lda % 4 == 0 && a_contig % 4 == 0 && (!batched || g.sA % 4 == 0);
  p.vec_b = aligned16(g.B) && g.ldb % 4 == 0 && b_contig % 4 == 0 && (!batched || g.sB % 4 == 0);
  p.vec_c = aligned16(g.C) && g.ldc % 4 == 0 && (!batched || g.sC % 4 == 0);
  const size_t gx = (g.m + BM - 1) / BM, gy = (g.n + BN - 1) / BN;
  if (gy > 65535 || g.batch > 65535) return MMBO_ERR_TOO_LARGE;
  dim3 grid((unsigned)gx, (unsigned)gy, (unsigned)g.batch), block((BM / TTM) * (BN / TTN));
  const float* A = static_cast<const float*>(g.A);
  const float* B = static_cast<const float*>(g.B);
  float* C = static_cast<float*>(g.C);
  if (!g.transA && !g.transB)
    sgemm_ffma_kernel<BM, BN, BK, TTM, TTN, false, false><<<grid, block, 0, st>>>(A, B, C, p);
  else if (!g.transA && g.transB)
    sgemm_ffma_kernel<BM, BN, BK, TTM, TTN, false, true><<<grid, block, 0, st>>>(A, B, C, p);
  else if (g.transA && !g.transB)
    sgemm_ffma_kernel<BM, BN, BK, TTM, TTN, true, false><<<grid, block, 0, st>>>(A, B, C, p);
  else
    sgemm_ffma_kernel<BM, BN, BK, TTM, TTN, true, true><<<grid, block, 0, st>>>(A, B, C, p);
  MMBO_COUNT_LAUNCH();
  return (int)cudaGetLastError();
}

// The tcgen05 kernel addresses its operands through TMA: 16-byte aligned bases and
// leading dimensions that are multiples of 8 fp16 elements.
static bool hgemm_tma_ok(const GemmArgs& g) {
  return aligned16(g.A) && aligned16(g.B) && g.lda % 8 == 0 && g.ldb % 8 == 0 && g.k > 0;
}

template <int TM, int STAGES, int CG, int EW, bool AK, bool BK_, int CSETS = (EW == 8 ? 2 : 1)>
static int launch_hgemm_inst(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
                             const HgemmParams& p, const HgemmPeerMaps& peers, uint64_t tiles, cudaStream_t st) {
  using L = HgemmSmem<TM, STAGES, CG, EW, CSETS>;
  auto kern = hgemm_tcgen05_kernel<TM, STAGES, AK, BK_, CG, EW, CSETS>;
  static bool attr_done[kMaxDevices] = {};
  static int max_walkers[kMaxDevices] = {};
  const int dev = current_device();
  if (dev < 0 || dev >= kMaxDevices) return MMBO_ERR_TOO_LARGE;
  if (!attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic);
    if (e != cudaSuccess) return (int)e;
    int walkers = sm_count() / CG;
    if (CG == 2) {
      // How many CTA pairs the device can hold at once (GPCs with an odd number of
      // SMs leave one SM unpaired).
      cudaLaunchConfig_t q = {};
      q.gridDim = dim3((unsigned)(2 * walkers));
      q.blockDim = dim3(L::kThreads);
      q.dynamicSmemBytes = L::kDynamic;
      cudaLaunchAttribute qa[1];
      qa[0].id = cudaLaunchAttributeClusterDimension;
      qa[0].val.clusterDim.x = 2; qa[0].val.clusterDim.y = 1; qa[0].val.clusterDim.z = 1;
      q.attrs = qa; q.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kern, &q) == cudaSuccess && n > 0) walkers = n < walkers ? n : walkers;
      else cudaGetLastError();
    }
    max_walkers[dev] = walkers;
    attr_done[dev] = true;
  }
  const unsigned walkers = (unsigned)(tiles < (uint64_t)max_walkers[dev] ? tiles : (uint64_t)max_walkers[dev]);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(walkers * CG);
  cfg.blockDim = dim3(L::kThreads);
  cfg.dynamicSmemBytes = L::kDynamic;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CG; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  // Programmatic dependent launch: the CTAs of this grid may become resident while the previous kernel of the
  // stream is still finishing; they initialise barriers and tensor memory, then wait (griddepcontrol.wait) for
  // that kernel to complete and flush before touching global memory.  Every CTA of the grid is resident at once
  // (persistent grid), so an early start of a dependent grid can never take an SM this grid still needs.
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = settings().pdl ? 2 : 1;
  MMBO_COUNT_LAUNCH();
  return (int)cudaLaunchKernelEx(&cfg, kern, ta, tb, tc, p, peers);
}

template <int TM, int STAGES, int CG, int EW = 4, int CSETS = (EW == 8 ? 2 : 1)>
static int launch_hgemm_tcgen05(const GemmArgs& g, uint32_t wgm, cudaStream_t st) {
  CUtensorMap ta, tb, tc;
  int rc;
  constexpr auto F16 = CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  constexpr auto SW = CU_TENSOR_MAP_SWIZZLE_128B;
  // C goes through staging buffers of kChunkRows rows x 32 columns, swizzled by their row length
  constexpr uint32_t kCR = HgemmSmem<TM, STAGES, CG, EW, CSETS>::kChunkRows;
  constexpr auto SWC = kCR == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  // op(A): K-major when transposed (stored k x m), MN-major otherwise (stored m x k).
  if (g.transA)
    rc = make_map(&ta, F16, 2, g.A, g.k, g.m, g.lda, kBlockK, HgemmSmem<TM, STAGES, CG, EW, CSETS>::kPieceRows, SW, g.batch, g.sA);
  else
    rc = make_map(&ta, F16, 2, g.A, g.m, g.k, g.lda, 64, kBlockK, SW, g.batch, g.sA);
  if (rc) return rc;
  // op(B): K-major when not transposed (stored k x n), MN-major otherwise (stored n x k).
  if (!g.transB)
    rc = make_map(&tb, F16, 2, g.B, g.k, g.n, g.ldb, kBlockK, kTileN, SW, g.batch, g.sB);
  else
    rc = make_map(&tb, F16, 2, g.B, g.n, g.k, g.ldb, 64, kBlockK, SW, g.batch, g.sB);
  if (rc) return rc;
  // C through TMA only when whole 16-byte units stay inside the matrix (see HgemmParams).
  const bool c_tma = aligned16(g.C) && g.ldc % 8 == 0 && g.m % 8 == 0 && batch_stride_ok(g.batch, g.sC, 2);
  if (c_tma) {
    rc = make_map(&tc, F16, 2, g.C, g.m, g.n, g.ldc, kCR, 32, SWC, g.batch, g.sC);
    if (rc) return rc;
  } else {
    tc = ta;  // placeholder, never dereferenced by the plain epilogue
  }
  static HgemmPeerMaps peers;  // (callers hold the library lock)
  peers.count = 0;
  if (g.npeers > 0) {
    // peer copies go through TMA stores only, and only for a single problem
    if (!c_tma || g.npeers > kMaxPeerCopies || g.batch != 1) return MMBO_ERR_KERNEL_UNSUITABLE;
    for (int d = 0; d < g.npeers; ++d) {
      if (!g.peers[d] || !aligned16(g.peers[d])) return MMBO_ERR_KERNEL_UNSUITABLE;
      rc = make_map_2d(&peers.map[d], F16, 2, g.peers[d], g.m, g.n, g.ldc, kCR, 32, SWC);
      if (rc) return rc;
    }
    peers.count = (uint32_t)g.npeers;
  }

  HgemmParams p;
  p.m = (uint32_t)g.m; p.n = (uint32_t)g.n; p.k = (uint32_t)g.k;
  p.tiles_m = (uint32_t)((g.m + TM - 1) / TM);
  p.tiles_n = (uint32_t)((g.n + kTileN * CG - 1) / (kTileN * CG));
  p.batch = (uint32_t)g.batch;
  p.c_batch_stride = g.sC;
  p.wgm = wgm;
  p.walk = mmbo_tile_walk_make(p.tiles_m, p.tiles_n, wgm);
  p.alpha = g.alpha; p.beta = g.beta;
  p.c = static_cast<__half*>(g.C); p.ldc = (uint32_t)g.ldc; p.c_tma = c_tma ? 1u : 0u;
  p.c_mc = nullptr;
  if (g.c_multicast) {
    // the multicast window is written with 16-byte stores of whole column pieces
    if (!c_tma || g.batch != 1 || !aligned16(g.c_multicast) || g.npeers > 0) return MMBO_ERR_KERNEL_UNSUITABLE;
    p.c_mc = static_cast<__half*>(g.c_multicast);
  }
  p.trace = g_trace_buffer;  // null unless mmbo_debug_trace armed it
  p.diag = settings().diag;  // diagnostic builds (no C store / no drain): never set in production
  const uint64_t tiles = (uint64_t)p.tiles_m * p.tiles_n * g.batch;
  if (tiles > 0x7fffffffull) return MMBO_ERR_TOO_LARGE;
  if (g.transA && !g.transB) return launch_hgemm_inst<TM, STAGES, CG, EW, true, true, CSETS>(ta, tb, tc, p, peers, tiles, st);
  if (g.transA && g.transB) return launch_hgemm_inst<TM, STAGES, CG, EW, true, false, CSETS>(ta, tb, tc, p, peers, tiles, st);
  if (!g.transA && !g.transB) return launch_hgemm_inst<TM, STAGES, CG, EW, false, true, CSETS>(ta, tb, tc, p, peers, tiles, st);
  return launch_hgemm_inst<TM, STAGES, CG, EW, false, false, CSETS>(ta, tb, tc, p, peers, tiles, st);
}

// Scratch layout of the 3xTF32 SGEMM: A_hi, A_lo (batch x m rows of Kpad floats), B_hi, B_lo (batch x n rows).
struct Tf32Scratch {
  size_t kpad, a_bytes, b_bytes, total;
};
static Tf32Scratch tf32_scratch(size_t m, size_t n, size_t k, size_t batch = 1) {
  Tf32Scratch s;
  s.kpad = align_up(k, 32);
  s.a_bytes = align_up(batch * m * s.kpad * 4, 1024);
  s.b_bytes = align_up(batch * n * s.kpad * 4, 1024);
  s.total = 2 * (s.a_bytes + s.b_bytes);
  return s;
}

template <int TM, int STAGES, int CG, int EW>
static int launch_tf32x3_gemm(const GemmArgs& g, const float* a_hi, const float* a_lo, const float* b_hi,
                              const float* b_lo, size_t kpad, uint32_t wgm, cudaStream_t st) {
  using L = TfSmem<TM, STAGES, CG, EW>;
  auto kern = sgemm_tf32x3_kernel<TM, STAGES, CG, EW>;
  CUtensorMap ta_hi, ta_lo, tb_hi, tb_lo, tc;
  int rc;
  constexpr auto F32 = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  constexpr auto SW = CU_TENSOR_MAP_SWIZZLE_128B;
  // packed operands of problem b start b * rows * kpad floats into their array
  if ((rc = make_map(&ta_hi, F32, 4, a_hi, g.k, g.m, kpad, kTfBlockK, TM / CG, SW, g.batch, g.m * kpad))) return rc;
  if ((rc = make_map(&ta_lo, F32, 4, a_lo, g.k, g.m, kpad, kTfBlockK, TM / CG, SW, g.batch, g.m * kpad))) return rc;
  if ((rc = make_map(&tb_hi, F32, 4, b_hi, g.k, g.n, kpad, kTfBlockK, kTfTileN, SW, g.batch, g.n * kpad))) return rc;
  if ((rc = make_map(&tb_lo, F32, 4, b_lo, g.k, g.n, kpad, kTfBlockK, kTfTileN, SW, g.batch, g.n * kpad))) return rc;
  // TMA stores whole 16-byte units: only when m is a multiple of 4 floats do they stay
  // inside the matrix.
  const bool c_tma = aligned16(g.C) && g.ldc % 4 == 0 && g.m % 4 == 0 && batch_stride_ok(g.batch, g.sC, 4);
  if (c_tma) {
    if ((rc = make_map(&tc, F32, 4, g.C, g.m, g.n, g.ldc, 32, 32, SW, g.batch, g.sC))) return rc;
  } else {
    tc = ta_hi;  // placeholder, never dereferenced by the plain epilogue
  }
  TfParams p;
  p.m = (uint32_t)g.m; p.n = (uint32_t)g.n; p.k = (uint32_t)g.k;
  p.tiles_m = (uint32_t)((g.m + TM - 1) / TM);
  p.tiles_n = (uint32_t)((g.n + kTfTileN * CG - 1) / (kTfTileN * CG));
  p.batch = (uint32_t)g.batch;
  p.c_batch_stride = g.sC;
  p.wgm = wgm; p.alpha = g.alpha; p.beta = g.beta;
  p.walk = mmbo_tile_walk_make(p.tiles_m, p.tiles_n, wgm);
  p.c = static_cast<float*>(g.C); p.ldc = (uint32_t)g.ldc; p.c_tma = c_tma ? 1u : 0u;
  p.chunk = settings().tf32_chunk;
  const uint64_t tiles = (uint64_t)p.tiles_m * p.tiles_n * g.batch;
  if (tiles > 0x7fffffffull) return MMBO_ERR_TOO_LARGE;

  static bool attr_done[kMaxDevices] = {};
  static int max_walkers[kMaxDevices] = {};
  const int dev = current_device();
  if (dev < 0 || dev >= kMaxDevices) return MMBO_ERR_TOO_LARGE;
  if (!attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic);
    if (e != cudaSuccess) return (int)e;
    int walkers = sm_count() / CG;
    if (CG == 2) {
      cudaLaunchConfig_t q = {};
      q.gridDim = dim3((unsigned)(2 * walkers));
      q.blockDim = dim3(L::kThreads);
      q.dynamicSmemBytes = L::kDynamic;
      cudaLaunchAttribute qa[1];
      qa[0].id = cudaLaunchAttributeClusterDimension;
      qa[0].val.clusterDim.x = 2; qa[0].val.clusterDim.y = 1; qa[0].val.clusterDim.z = 1;
      q.attrs = qa; q.numAttrs = 1;
      int nmax = 0;
      if (cudaOccupancyMaxActiveClusters(&nmax, kern, &q) == cudaSuccess && nmax > 0) walkers = nmax < walkers ? nmax : walkers;
      else cudaGetLastError();
    }
    max_walkers[dev] = walkers;
    attr_done[dev] = true;
  }
  const unsigned walkers = (unsigned)(tiles < (uint64_t)max_walkers[dev] ? tiles : (uint64_t)max_walkers[dev]);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(walkers * CG);
  cfg.blockDim = dim3(L::kThreads);
  cfg.dynamicSmemBytes = L::kDynamic;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CG; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // (as for the fp16 kernels)
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = settings().pdl ? 2 : 1;
  MMBO_COUNT_LAUNCH();
  return (int)cudaLaunchKernelEx(&cfg, kern, ta_hi, ta_lo, tb_hi, tb_lo, tc, p);
}

// Split + repack of both operands into `scratch`, then the tensor-core GEMM.
template <int TM, int STAGES, int CG, int EW = 4>
static int run_tf32x3(const GemmArgs& g, void* scratch, uint32_t wgm, cudaStream_t st) {
  const Tf32Scratch s = tf32_scratch(g.m, g.n, g.k, g.batch);
  if (((g.m + 63) / 64) > 65535 || ((g.n + 63) / 64) > 65535 || g.batch > 65535) return MMBO_ERR_TOO_LARGE;
  char* base = static_cast<char*>(scratch);
  float* a_hi = reinterpret_cast<float*>(base);
  float* a_lo = reinterpret_cast<float*>(base + s.a_bytes);
  float* b_hi = reinterpret_cast<float*>(base + 2 * s.a_bytes);
  float* b_lo = reinterpret_cast<float*>(base + 2 * s.a_bytes + s.b_bytes);
  const dim3 block(256);
  const dim3 grid_a((unsigned)((g.k + 63) / 64), (unsigned)((g.m + 63) / 64), (unsigned)g.batch);
  const dim3 grid_b((unsigned)((g.k + 63) / 64), (unsigned)((g.n + 63) / 64), (unsigned)g.batch);
  const float* A = static_cast<const float*>(g.A);
  const float* B = static_cast<const float*>(g.B);
  // op(A)(i,l): row index contiguous unless transposed; op(B)(l,j) as an n x k operand:
  // row index contiguous when transposed.
  if (!g.transA) split_pack_kernel<true><<<grid_a, block, 0, st>>>(A, g.lda, (uint32_t)g.m, (uint32_t)g.k, (uint32_t)s.kpad, a_hi, a_lo, g.sA);
  else split_pack_kernel<false><<<grid_a, block, 0, st>>>(A, g.lda, (uint32_t)g.m, (uint32_t)g.k, (uint32_t)s.kpad, a_hi, a_lo, g.sA);
  MMBO_COUNT_LAUNCH();
  if (g.transB) split_pack_kernel<true><<<grid_b, block, 0, st>>>(B, g.ldb, (uint32_t)g.n, (uint32_t)g.k, (uint32_t)s.kpad, b_hi, b_lo, g.sB);
  else split_pack_kernel<false><<<grid_b, block, 0, st>>>(B, g.ldb, (uint32_t)g.n, (uint32_t)g.k, (uint32_t)s.kpad, b_hi, b_lo, g.sB);
  MMBO_COUNT_LAUNCH();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  return launch_tf32x3_gemm<TM, STAGES, CG, EW>(g, a_hi, a_lo, b_hi, b_lo, s.kpad, wgm, st);
}

// ------------------------------------------------------------------ tuning table -----
// Exact-size overrides of the selection heuristics, the counterpart of the reference's
// Tensile library logic (src/gemm/ref/vega20_Cijk_Ailk_Bjlk_DB.yaml:929-1177: one
// [size] -> [solution index, GFLOP/s] row per tuned problem).  Rows come from
// mmbo_tuning_set, from a file given to mmbo_tuning_load, or from the file named by the
// environment variable MMBO_TUNING_FILE (read once, on the first automatic selection).
// File format, one row per line, '#' starts a comment:
//     <dtype f16|f32|f64> <trans NN|NT|TN|TT> <m> <n> <k> <kernelId> [<split>]
// split (optional, default 0): how the contraction is split for this problem -- 0 decided per call, 1 never,
// 2 always (stream-K, rows that have it) -- the counterpart of a tuned GlobalSplitU value
// (src/gemm/ref/vega20_Cijk_Ailk_Bjlk_DB.yaml:69-71).
struct TuneRow {
  int dtype, ta, tb;
  size_t m, n, k;
  int kernel;
  int split;
};
constexpr int kMaxTuneRows = 4096;
static TuneRow g_tune[kMaxTuneRows];
static int g_tune_count = 0;
static bool g_tune_env_done = false;

static int tune_set(int dtype, int ta, int tb, size_t m, size_t n, size_t k, int kernel, int split = 0) {
  int count = 0;
  if (!rows_of(dtype, &count)) return MMBO_ERR_BAD_DTYPE;
  if (kernel < 0 || kernel >= count) return MMBO_ERR_BAD_KERNEL_ID;
  if (split < 0 || split > 2) return MMBO_ERR_BAD_OPTION;
  for (int i = 0; i < g_tune_count; ++i) {
    TuneRow& r = g_tune[i];
    if (r.dtype == dtype && r.ta == ta && r.tb == tb && r.m == m && r.n == n && r.k == k) {
      r.kernel = kernel;
      r.split = split;
      return MMBO_OK;
    }
  }
  if (g_tune_count >= kMaxTuneRows) return MMBO_ERR_TOO_LARGE;
  g_tune[g_tune_count++] = TuneRow{dtype, ta, tb, m, n, k, kernel, split};
  return MMBO_OK;
}

static int tune_load(const char* path) {
  FILE* f = fopen(path, "r");
  if (!f) return MMBO_ERR_TUNING_FILE;
  char line[256];
  int rc = MMBO_OK;
  while (fgets(line, sizeof line, f)) {
    char dt[8], tr[8];
    unsigned long long m, n, k;
    int kernel, split = 0;
    if (line[0] == '#' || line[0] == '\n') continue;
    if (sscanf(line, "%7s %7s %llu %llu %llu %d %d", dt, tr, &m, &n, &k, &kernel, &split) < 6) { rc = MMBO_ERR_TUNING_FILE; break; }
    const int dtype = !strcmp(dt, "f16") ? MMBO_DTYPE_F16 : !strcmp(dt, "f32") ? MMBO_DTYPE_F32
                      : !strcmp(dt, "f64") ? MMBO_DTYPE_F64 : -1;
    if (dtype < 0 || strlen(tr) != 2) { rc = MMBO_ERR_TUNING_FILE; break; }
    rc = tune_set(dtype, tr[0] == 'T', tr[1] == 'T', m, n, k, kernel, split);
    if (rc) { rc = MMBO_ERR_TUNING_FILE; break; }
  }
  fclose(f);
  return rc;
}

// Kernel id the table holds for this exact problem, or -1.
static int tune_lookup(int dtype, const GemmArgs& g) {
  if (!g_tune_env_done) {
    g_tune_env_done = true;
    const char* path = getenv("MMBO_TUNING_FILE");
    if (path && *path) tune_load(path);
  }
  for (int i = 0; i < g_tune_count; ++i) {
    const TuneRow& r = g_tune[i];
    if (r.dtype == dtype && r.ta == g.transA && r.tb == g.transB && r.m == g.m && r.n == g.n && r.k == g.k) {
      g_split_from_table = (uint32_t)r.split;
      return r.kernel;
    }
  }
  return -1;
}

// ------------------------------------------------------------------ selection --------
// Exact fp32 (CUDA-core FFMA) choice: the producer / consumer kernel from two tiles per SM on
// (2048^3: 51.0 against 45.8 TFLOP/s for id 1, 4096^3: 61.1 / 55.5, 8192^3: 61.4 / 56.6); the
// 64 x 64 kernel below that (1024^3: 30.6 against 23.0).
static int select_f32_exact(const GemmArgs& g) {
  const uint64_t big_tiles = (uint64_t)((g.m + 127) / 128) * ((g.n + 127) / 128) * g.batch;
  return big_tiles >= 2ull * (uint64_t)sm_count() ? 6 : 2;
}

static int select_f32(const GemmArgs& g) {
  if (g.k == 0) return 0;
  const bool exact = settings().f32_exact != 0;
  const int tuned = tune_lookup(MMBO_DTYPE_F32, g);
  // A tuned row that names a split-precision tensor-core kernel is ignored when the caller asked
  // for exact fp32 arithmetic: the switch is a statement about numerics, the table one about speed.
  if (tuned >= 0 && !(exact && kF32Rows[tuned].tensor)) return tuned;
  // The split-precision tensor-core kernels hold the fp32 tolerance and are several
  // times faster than the FFMA pipe once the three launches they need are amortised.
  // MMBO_F32_EXACT=1 keeps automatic selection on the CUDA-core kernels.
  const double work = (double)g.m * (double)g.n * (double)g.k * (double)g.batch;
  if (work >= 512.0 * 512.0 * 512.0 && !exact) {
    const uint64_t big_pairs = (uint64_t)((g.m + 255) / 256) * ((g.n + 255) / 256) * g.batch;
    // 256 x 256 pair tiles from 48 of them on (measured by the autotuner: 2048^3 173 against 134 TFLOP/s for the
    // 128 x 256 row, 2368^3 148 / 135, 3072^3 231 / 178, 1536 x 2048 x 384 (48 tiles) 73 / 63; but 1536^3 (36 tiles)
    // 105 against 133 for the 128 x 128 row)
    if (big_pairs >= 48) return 5;
    const uint64_t pair_tiles = (uint64_t)((g.m + 127) / 128) * ((g.n + 255) / 256) * g.batch;
    return pair_tiles >= (uint64_t)(sm_count() / 2) ? 3 : 4;
  }
  return select_f32_exact(g);
}

static int select_f16(const GemmArgs& g) {
  if (g.k == 0) return 0;
  const int tuned = tune_lookup(MMBO_DTYPE_F16, g);
  if (tuned >= 0) return tuned;
  // Operands TMA cannot address are realigned through scratch first; that only pays off
  // once the product dwarfs the copies.
  if (!hgemm_tma_ok(g) && (double)g.m * (double)g.n * (double)g.k < 256.0 * 256.0 * 256.0) return 0;
  const uint64_t nb = g.batch;  // every problem of a strided batch adds its tiles to the walk
  // Score = fraction of the machine kept busy over whole waves of tiles x relative
  // speed of the kernel on a full wave (measured on 8192^3).
  const double sms = (double)sm_count();
  auto eff = [](uint64_t tiles, double walkers) {
    const double waves = (double)((tiles + (uint64_t)walkers - 1) / (uint64_t)walkers);
    return (double)tiles / (waves * walkers);
  };
  const uint64_t t1 = nb * ((g.m + 255) / 256) * ((g.n + 127) / 128);
  const uint64_t t2 = nb * ((g.m + 127) / 128) * ((g.n + 127) / 128);
  const uint64_t t3 = nb * ((g.m + 255) / 256) * ((g.n + 255) / 256);
  // useful fraction of each tile (ragged edges waste tensor work)
  auto fill = [&](uint64_t tiles, double tm, double tn) { return ((double)nb * (double)g.m * (double)g.n) / ((double)tiles * tm * tn); };
  const double s1 = 0.80 * eff(t1, sms) * fill(t1, 256, 128);
  const double s2 = 0.70 * eff(t2, sms) * fill(t2, 128, 128);
  const double s3 = 1.00 * eff(t3, sms / 2) * fill(t3, 256, 256);
  // 512-row pair tiles: 25 % less operand staging per flop (8192^3: 1404 against 1358 TFLOP/s; seconds-long loops
  // under the power cap: 1306 against 1257, at a higher clock), but a single accumulator, so the epilogue is
  // not hidden: only for long contractions (8192 x 8192 x 4096: 432 against 404 us for the 256-row row; x 8192:
  // 719-796 against 756-833).
  const uint64_t t6 = nb * ((g.m + 511) / 512) * ((g.n + 255) / 256);
  const double s6 = 1.03 * eff(t6, sms / 2) * fill(t6, 512, 256);
  if (g.k >= 6144 && s6 >= s3 && s6 >= s1 && s6 >= s2) return 6;
  // Short contractions are bound by the epilogue: the rows with eight epilogue warps win there (measured on
  // 8192 x 8192 x k, TN, us; rows 4 / 5 / 3):
  //   beta == 0:  k = 256: 43.6 / 40.4 / 55.5   512: 69.9 / 62.2 / 65.8   1024: 119 / 105.7 / 102.1   2048: 228 / 201 / 190-207
  //   beta != 0:  k = 256: 59.7 / 62.0 / 99.2   512: 83.7 / 77.1 / 105    1024: 141 / 124.3 / 143.5   2048: 272 / 217 / 206
  // Row 4 requests the old C a whole tile ahead into a second set of staging buffers (three operand stages): it
  // pays only while a tile's main loop is shorter than the latency of that request.  Row 5 has five stages and an
  // L2 prefetch of the next tile's C instead; the six-stage row with four epilogue warps takes over once the main
  // loop hides the epilogue.
  if (s3 >= s1 && s3 >= s2) {
    // At most two tiles per CTA pair: the last epilogue is not hidden behind anything, and eight epilogue warps
    // finish it sooner (autotuner, beta = 0.5: 2048^3 874 against 798 TFLOP/s, 2368^3 783 against 753).
    if (t3 <= 2 * (uint64_t)(sms / 2) && g.k <= 4096) return (g.k <= 256 && g.beta != 0.0f) ? 4 : 5;
    if (g.beta != 0.0f) return g.k <= 256 ? 4 : (g.k <= 1536 ? 5 : 3);
    return g.k < 1024 ? 5 : 3;
  }
  return s1 >= s2 ? 1 : 2;
}

// Automatic selection for a call that is about to run: a split-precision row whose scratch
// does not fit the buffer the caller lent falls back to the CUDA-core kernels instead of failing.
static int select_f32_fitting(const GemmArgs& g) {
  const int id = select_f32(g);
  if (id >= 3 && id <= 5) {
    const int dev = current_device();
    if (dev >= 0 && dev < kMaxDevices && g_ws[dev].user && g_ws[dev].bytes < tf32_scratch(g.m, g.n, g.k, g.batch).total)
      return select_f32_exact(g);
  }
  return id;
}

static int g_last_kernel[3] = {-1, -1, -1};  // row the last call of each dtype ran (mmbo_last_kernel)

static int run_f32(const GemmArgs& g, int id, cudaStream_t st) {
  g_last_kernel[MMBO_DTYPE_F32] = id;
  if (g.m == 0 || g.n == 0) return MMBO_OK;
  if (g.k == 0) return launch_scale<float>(g, st);
  switch (id) {
    case 0: return launch_simple<float>(g, st);
    case 1: return launch_sgemm_ffma<128, 128, 8, 8>(g, wgm_of(kF32Rows[1]), st);
    case 2: return launch_sgemm_ffma<64, 64, 4, 4>(g, wgm_of(kF32Rows[2]), st);
    case 6: return launch_sgemm_ffma_ws(g, wgm_of(kF32Rows[6]), st);
    case 3:
    case 4:
    case 5: {
      void* scratch = nullptr;
      int rc = ensure_workspace(tf32_scratch(g.m, g.n, g.k, g.batch).total, &scratch);
      if (rc) return rc;
      if ((rc = workspace_acquire(st))) return rc;
      if (id == 3) rc = run_tf32x3<128, 4, 2>(g, scratch, wgm_of(kF32Rows[3]), st);
      else if (id == 5) rc = run_tf32x3<256, 3, 2, 8>(g, scratch, wgm_of(kF32Rows[5]), st);
      else rc = run_tf32x3<128, 3, 1>(g, scratch, wgm_of(kF32Rows[4]), st);
      const int rc2 = workspace_release(st);
      return rc ? rc : rc2;
    }
  }
  return MMBO_ERR_BAD_KERNEL_ID;
}

// Default fp64 kernel: the warp-specialised tensor kernel.  64-row tiles for short contractions
// (the epilogue weighs more and more CTAs overlap it: 32.4 against 32.2 TFLOP/s at 44160 x 2048 x 384,
// 31.8 / 30.1 at 11136, 17.2 / 14.7 at 384) and while 128-row tiles would not give every CTA slot
// of the machine a tile (1024^3: 28.3 / 23.7); 128-row tiles otherwise (3072^3: 34.8 / 34.3).
static int select_f64(const GemmArgs& g) {
  const size_t slots = 2 * (size_t)sm_count();  // CTAs resident at once
  const size_t tiles128 = g.batch * ((g.m + 127) / 128) * ((g.n + kWsBN - 1) / kWsBN);
  const size_t tiles64 = g.batch * ((g.m + 63) / 64) * ((g.n + kWsBN - 1) / kWsBN);
  if (g.k <= 512) return 4;
  // Longer contractions: estimated time of each tile height in slabs of a 64-row tile -- whole rounds of the
  // CTA slots, or the even split of stream-K where that applies (plan_stream_k) -- the 64-row tiles being
  // about 1.5 % slower per unit of work (3072^3: 34.8 / 34.3 TFLOP/s).  Without stream-K the tile height whose
  // tile count fills whole rounds better wins (2368^3 with 128-row tiles: 703 tiles = 2.4 rounds, 27.4 TFLOP/s
  // against 34.4 at 2176^3 = 1.95 rounds).
  const size_t num_kb = (g.k + kWsBK - 1) / kWsBK;
  auto slabs = [&](size_t tiles, size_t bm) {
    const SkPlan pl = plan_stream_k(tiles, num_kb, slots, bm * kWsBN * 8, kWsConsumers, g.batch);
    if (pl.on) return (double)tiles * (double)num_kb / (double)pl.grid + 6.0;
    return (double)((tiles + slots - 1) / slots) * (double)num_kb;
  };
  return 1.015 * slabs(tiles64, 64) < 2.0 * slabs(tiles128, 128) ? 4 : 3;
}

static int run_f64(const GemmArgs& g, double alpha, double beta, int id, cudaStream_t st) {
  g_last_kernel[MMBO_DTYPE_F64] = id;
  if (g.m == 0 || g.n == 0) return MMBO_OK;
  const double* A = static_cast<const double*>(g.A);
  const double* B = static_cast<const double*>(g.B);
  double* C = static_cast<double*>(g.C);
  if (g.batch > 65535) return MMBO_ERR_TOO_LARGE;
  if (g.k == 0 || id == 0) {
    const size_t gx = (g.m + 31) / 32, gy = (g.n + 7) / 8;
    if (gy > 65535 || gx > 0x7fffffffull) return MMBO_ERR_TOO_LARGE;
    dim3 grid((unsigned)gx, (unsigned)gy, (unsigned)g.batch), block(32, 8);
    if (g.k == 0) scale_c_f64_kernel<<<grid, block, 0, st>>>(g.m, g.n, beta, C, g.ldc, g.sC);
    else gemm_simple_f64_kernel<<<grid, block, 0, st>>>(g.transA, g.transB, g.m, g.n, g.k, alpha, A, g.lda, B, g.ldb, beta, C, g.ldc,
                                                         g.sA, g.sB, g.sC);
    MMBO_COUNT_LAUNCH();
    return (int)cudaGetLastError();
  }
  if (id < 1 || id > 4) return MMBO_ERR_BAD_KERNEL_ID;
  DgemmParams p;
  p.m = (uint32_t)g.m; p.n = (uint32_t)g.n; p.k = (uint32_t)g.k;
  p.lda = (uint32_t)g.lda; p.ldb = (uint32_t)g.ldb; p.ldc = (uint32_t)g.ldc;
  p.alpha = alpha; p.beta = beta; p.wgm = wgm_of(kF64Rows[id]);
  p.diag = settings().diag;
  p.tma_a = p.tma_b = p.tma_c = 0;
  p.batch = (uint32_t)g.batch;
  p.batch_a = g.sA; p.batch_b = g.sB; p.batch_c = g.sC;
  if (id == 2) {  // fp64 tensor path
    const size_t gx2 = (g.m + kDmBM - 1) / kDmBM, gy2 = (g.n + kDmBN - 1) / kDmBN;
    if (gy2 > 65535) return MMBO_ERR_TOO_LARGE;
    dim3 grid2((unsigned)gx2, (unsigned)gy2, (unsigned)g.batch);
    if (!g.transA && !g.transB) dgemm_dmma_kernel<false, false><<<grid2, kDmThreads, 0, st>>>(A, B, C, p);
    else if (!g.transA && g.transB) dgemm_dmma_kernel<false, true><<<grid2, kDmThreads, 0, st>>>(A, B, C, p);
    else if (g.transA && !g.transB) dgemm_dmma_kernel<true, false><<<grid2, kDmThreads, 0, st>>>(A, B, C, p);
    else dgemm_dmma_kernel<true, true><<<grid2, kDmThreads, 0, st>>>(A, B, C, p);
    MMBO_COUNT_LAUNCH();
    return (int)cudaGetLastError();
  }
  if (id == 3 || id == 4) {  // fp64 tensor path, producer and consumer warpgroups, persistent; 128- or 64-row tiles
    const size_t bm = id == 3 ? 128 : 64;
    const size_t tiles = ((g.m + bm - 1) / bm) * ((g.n + kWsBN - 1) / kWsBN) * g.batch;
    if (tiles > 0x7fffffffull) return MMBO_ERR_TOO_LARGE;
    unsigned grid3 = (unsigned)std::min(tiles, (size_t)2 * (size_t)sm_count());  // two CTAs per SM (more made no difference)
    const SkPlan plan = plan_stream_k(tiles, (g.k + kWsBK - 1) / kWsBK, (size_t)2 * (size_t)sm_count(), bm * kWsBN * 8,
                                      kWsConsumers, g.batch);
    StreamK sk;
    {
      const int rc = prepare_stream_k(plan, st, &sk);
      if (rc == MMBO_OK && plan.on) grid3 = plan.grid;
      else sk.enabled = 0;  // no scratch to be had (a lent buffer that is too small): whole tiles
    }
    // An operand goes through TMA when its base is 16-byte aligned and its leading dimension even
    // (strides in multiples of 16 bytes); the box is kWsPad elements wider than the tile along the
    // contiguous index, which gives the slab its padded pitch.
    CUtensorMap ta, tb;
    constexpr auto F64 = CU_TENSOR_MAP_DATA_TYPE_FLOAT64;
    constexpr auto NOSW = CU_TENSOR_MAP_SWIZZLE_NONE;
    p.tma_a = aligned16(g.A) && g.lda % 2 == 0 && batch_stride_ok(g.batch, g.sA, 8);
    p.tma_b = aligned16(g.B) && g.ldb % 2 == 0 && batch_stride_ok(g.batch, g.sB, 8);
    if (p.tma_a) {
      const int rc = g.transA  // stored k x m (k contiguous) / m x k (m contiguous)
          ? make_map(&ta, F64, 8, g.A, g.k, g.m, g.lda, kWsBK + kWsPad, (uint32_t)bm, NOSW, g.batch, g.sA)
          : make_map(&ta, F64, 8, g.A, g.m, g.k, g.lda, (uint32_t)bm + kWsPad, kWsBK, NOSW, g.batch, g.sA);
      if (rc) return rc;
    } else {
      memset(&ta, 0, sizeof(ta));
    }
    if (p.tma_b) {
      const int rc = g.transB  // stored n x k (n contiguous) / k x n (k contiguous)
          ? make_map(&tb, F64, 8, g.B, g.n, g.k, g.ldb, kWsBN + kWsPad, kWsBK, NOSW, g.batch, g.sB)
          : make_map(&tb, F64, 8, g.B, g.k, g.n, g.ldb, kWsBK + kWsPad, kWsBN, NOSW, g.batch, g.sB);
      if (rc) return rc;
    } else {
      memset(&tb, 0, sizeof(tb));
    }
    // old C staged through shared memory (64-row tiles only): one box of 64 columns x (64 + 4) rows
    CUtensorMap tc;
    p.tma_c = id == 4 && beta != 0.0 && aligned16(g.C) && g.ldc % 2 == 0 && settings().dgemm_stage_c != 0 &&
              batch_stride_ok(g.batch, g.sC, 8);
    if (p.tma_c) {
      const int rc = make_map(&tc, F64, 8, g.C, g.m, g.n, g.ldc, (uint32_t)bm + kWsPad, kWsBN, NOSW, g.batch, g.sC);
      if (rc) return rc;
    } else {
      memset(&tc, 0, sizeof(tc));
    }
    auto launch = [&](auto kernel, size_t smem) -> int {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
      kernel<<<grid3, kWsThreads, smem, st>>>(ta, tb, tc, A, B, C, p, sk);
      MMBO_COUNT_LAUNCH();
      int rc = (int)cudaGetLastError();
      if (sk.enabled) {
        const int rc2 = workspace_release(st);
        if (!rc) rc = rc2;
      }
      return rc;
    };
    auto by_tile = [&](auto ta_, auto tb_) -> int {
      constexpr bool TA = decltype(ta_)::value, TB = decltype(tb_)::value;
      if (sk.enabled) {
        if (id == 3) return launch(dgemm_dmma_ws_kernel<TA, TB, 128, true>, WsTile<128, TA, !TB>::kSmemBytes);
        return launch(dgemm_dmma_ws_kernel<TA, TB, 64, true>, WsTile<64, TA, !TB>::kSmemBytes);
      }
      if (id == 3) return launch(dgemm_dmma_ws_kernel<TA, TB, 128>, WsTile<128, TA, !TB>::kSmemBytes);
      return launch(dgemm_dmma_ws_kernel<TA, TB, 64>, WsTile<64, TA, !TB>::kSmemBytes);
    };
    using Yes = std::true_type;
    using No = std::false_type;
    if (!g.transA && !g.transB) return by_tile(No{}, No{});
    if (!g.transA && g.transB) return by_tile(No{}, Yes{});
    if (g.transA && !g.transB) return by_tile(Yes{}, No{});
    return by_tile(Yes{}, Yes{});
  }
  const size_t gx = (g.m + kDgBM - 1) / kDgBM, gy = (g.n + kDgBN - 1) / kDgBN;
  if (gy > 65535) return MMBO_ERR_TOO_LARGE;
  dim3 grid((unsigned)gx, (unsigned)gy, (unsigned)g.batch);
  if (!g.transA && !g.transB) dgemm_fma_kernel<false, false><<<grid, kDgThreads, 0, st>>>(A, B, C, p);
  else if (!g.transA && g.transB) dgemm_fma_kernel<false, true><<<grid, kDgThreads, 0, st>>>(A, B, C, p);
  else if (g.transA && !g.transB) dgemm_fma_kernel<true, false><<<grid, kDgThreads, 0, st>>>(A, B, C, p);
  else dgemm_fma_kernel<true, true><<<grid, kDgThreads, 0, st>>>(A, B, C, p);
  MMBO_COUNT_LAUNCH();
  return (int)cudaGetLastError();
}

// fp16 operands TMA cannot address (base not 16-byte aligned or leading dimension not a
// multiple of 8) are first copied, column by column, into scratch with an aligned pitch
// (a strided device-to-device copy, no arithmetic), then the tensor-core kernel runs on
// the copies.  C needs no copy: the epilogue without TMA handles any C.
static int realign_f16(GemmArgs& g, cudaStream_t st, bool* scratch_used) {
  const bool a_ok = aligned16(g.A) && g.lda % 8 == 0, b_ok = aligned16(g.B) && g.ldb % 8 == 0;
  *scratch_used = false;
  if (a_ok && b_ok) return MMBO_OK;
  const size_t rowsA = g.transA ? g.k : g.m, colsA = g.transA ? g.m : g.k;
  const size_t rowsB = g.transB ? g.n : g.k, colsB = g.transB ? g.k : g.n;
  const size_t nlda = align_up(rowsA, 8), nldb = align_up(rowsB, 8);
  const size_t a_bytes = a_ok ? 0 : align_up(nlda * colsA * 2, 1024);
  const size_t b_bytes = b_ok ? 0 : align_up(nldb * colsB * 2, 1024);
  void* scratch = nullptr;
  int rc = ensure_workspace(a_bytes + b_bytes, &scratch);
  if (rc) return rc;
  if ((rc = workspace_acquire(st))) return rc;
  *scratch_used = true;
  char* base = static_cast<char*>(scratch);
  cudaError_t e;
  if (!a_ok) {
    e = cudaMemcpy2DAsync(base, nlda * 2, g.A, g.lda * 2, rowsA * 2, colsA, cudaMemcpyDeviceToDevice, st);
    if (e != cudaSuccess) return (int)e;
    g.A = base;
    g.lda = nlda;
  }
  if (!b_ok) {
    e = cudaMemcpy2DAsync(base + a_bytes, nldb * 2, g.B, g.ldb * 2, rowsB * 2, colsB, cudaMemcpyDeviceToDevice, st);
    if (e != cudaSuccess) return (int)e;
    g.B = base + a_bytes;
    g.ldb = nldb;
  }
  return MMBO_OK;
}

static int run_f16(const GemmArgs& g_in, int id, cudaStream_t st) {
  g_last_kernel[MMBO_DTYPE_F16] = id;
  if (g_in.m == 0 || g_in.n == 0) return MMBO_OK;
  if (g_in.k == 0) return launch_scale<__half>(g_in, st);
  if (id == 0) return launch_simple<__half>(g_in, st);
  if (id < 0 || id >= kNumF16) return MMBO_ERR_BAD_KERNEL_ID;
  GemmArgs g = g_in;
  bool scratch_used = false;
  int rc = realign_f16(g, st, &scratch_used);
  if (rc) return rc;
  switch (id) {
    case 1: rc = launch_hgemm_tcgen05<256, 4, 1>(g, wgm_of(kF16Rows[1]), st); break;
    case 2: rc = launch_hgemm_tcgen05<128, 6, 1>(g, wgm_of(kF16Rows[2]), st); break;
    case 3: rc = launch_hgemm_tcgen05<256, 6, 2>(g, wgm_of(kF16Rows[3]), st); break;
    case 4: rc = launch_hgemm_tcgen05<256, 3, 2, 8>(g, wgm_of(kF16Rows[4]), st); break;
    case 5: rc = launch_hgemm_tcgen05<256, 5, 2, 8, 1>(g, wgm_of(kF16Rows[5]), st); break;
    case 6: rc = launch_hgemm_tcgen05<512, 4, 2, 4>(g, wgm_of(kF16Rows[6]), st); break;
    case 7: rc = launch_hgemm_tcgen05<512, 4, 2, 8, 1>(g, wgm_of(kF16Rows[7]), st); break;
    default: rc = MMBO_ERR_BAD_KERNEL_ID;
  }
  if (scratch_used) {
    const int rc2 = workspace_release(st);
    if (!rc) rc = rc2;
  }
  return rc;
}

// ------------------------------------------------------------------ host operands ----
// GEMM on operands that live in HOST memory (what the reference's harness does by hand
// around its kernel: hipMalloc + hipMemcpy in, launch, hipMemcpy out --
// src/gemm/benchmark.cc:57-63, src/gemm/test.cc:53-66,89).  A is copied once; B and C
// travel in column panels through two device buffers each, so that the copy-in of panel
// j+1, the GEMM of panel j and the copy-out of panel j-1 overlap on three streams.
struct HostPipe {
  bool ready;
  cudaStream_t s_in, s_mm, s_out, s_cc;  // copy in, GEMM, copy out, collectives (sharded A)
  cudaEvent_t ev_a, ev_cc, ev_in[2], ev_mm[2], ev_out[2];
  void* buf;
  size_t bytes;
};
static HostPipe g_pipe[kMaxDevices];

static int pipe_setup(HostPipe& hp, size_t bytes) {
  cudaError_t e;
  if (!hp.ready) {
    if ((e = cudaStreamCreateWithFlags(&hp.s_in, cudaStreamNonBlocking)) != cudaSuccess) return (int)e;
    if ((e = cudaStreamCreateWithFlags(&hp.s_mm, cudaStreamNonBlocking)) != cudaSuccess) return (int)e;
    if ((e = cudaStreamCreateWithFlags(&hp.s_out, cudaStreamNonBlocking)) != cudaSuccess) return (int)e;
    if ((e = cudaStreamCreateWithFlags(&hp.s_cc, cudaStreamNonBlocking)) != cudaSuccess) return (int)e;
    cudaEventCreateWithFlags(&hp.ev_a, cudaEventDisableTiming);
    cudaEventCreateWithFlags(&hp.ev_cc, cudaEventDisableTiming);
    for (int i = 0; i < 2; ++i) {
      cudaEventCreateWithFlags(&hp.ev_in[i], cudaEventDisableTiming);
      cudaEventCreateWithFlags(&hp.ev_mm[i], cudaEventDisableTiming);
      cudaEventCreateWithFlags(&hp.ev_out[i], cudaEventDisableTiming);
    }
    hp.ready = true;
  }
  if (hp.bytes < bytes) {
    if (hp.buf) cudaFree(hp.buf);
    hp.buf = nullptr;
    hp.bytes = 0;
    if ((e = cudaMalloc(&hp.buf, bytes)) != cudaSuccess) return (int)e;
    hp.bytes = bytes;
  }
  return MMBO_OK;
}

// A replicated over the GPUs of a node without every rank pushing all of it through the host
// bridge: rank r copies only its share of A's stored columns host -> device, then the shares
// are exchanged over NVLink (ncclAllGather in place when the shares are equal, one grouped
// ncclBroadcast per rank otherwise).
struct ShardedA {
  int n_gpus, rank;
  void* comm;  // ncclComm_t of the caller
};

static int stage_a_sharded(const ShardedA& sa, HostPipe& hp, const GemmArgs& h, size_t es, char* dA, size_t dlda,
                           size_t rowsA, size_t colsA) {
  NcclApi& nc = nccl_api();
  if (!nc.ok()) return MMBO_ERR_NO_NCCL;
  const size_t al = 16 / es;  // shares start on 16-byte boundaries of the compact device layout
  size_t c0 = 0, cn = 0;
  int rc = mmbo_shard_columns(colsA, sa.n_gpus, sa.rank, al, &c0, &cn);
  if (rc) return rc;
  cudaError_t e;
  if (cn > 0) {
    e = cudaMemcpy2DAsync(dA + c0 * dlda * es, dlda * es, static_cast<const char*>(h.A) + c0 * h.lda * es, h.lda * es,
                          rowsA * es, cn, cudaMemcpyHostToDevice, hp.s_in);
    if (e != cudaSuccess) return (int)e;
  }
  cudaEventRecord(hp.ev_a, hp.s_in);
  cudaStreamWaitEvent(hp.s_cc, hp.ev_a, 0);
  bool equal = colsA % ((size_t)sa.n_gpus * al) == 0;
  int nrc = 0;
  if (equal) {
    nrc = nc.all_gather(dA + c0 * dlda * es, dA, cn * dlda * es, kNcclUint8, sa.comm, hp.s_cc);
  } else {
    nrc = nc.group_start();
    for (int r = 0; !nrc && r < sa.n_gpus; ++r) {
      size_t r0 = 0, rn = 0;
      mmbo_shard_columns(colsA, sa.n_gpus, r, al, &r0, &rn);
      if (rn == 0) continue;
      char* piece = dA + r0 * dlda * es;
      nrc = nc.broadcast(piece, piece, rn * dlda * es, kNcclUint8, r, sa.comm, hp.s_cc);
    }
    const int end = nc.group_end();
    if (!nrc) nrc = end;
  }
  if (nrc) return MMBO_ERR_NCCL;
  cudaEventRecord(hp.ev_cc, hp.s_cc);
  cudaStreamWaitEvent(hp.s_mm, hp.ev_cc, 0);  // the first GEMM needs all of A
  return MMBO_OK;
}

static int gemm_host(int dtype, const GemmArgs& h, int kernelId, double alpha64 = 0.0, double beta64 = 0.0,
                     const ShardedA* sharded_a = nullptr) {
  const size_t es = dtype == MMBO_DTYPE_F64 ? 8 : dtype == MMBO_DTYPE_F32 ? 4 : 2;
  const int dev = current_device();
  if (dev < 0 || dev >= kMaxDevices) return MMBO_ERR_TOO_LARGE;
  if (h.m == 0 || h.n == 0) return MMBO_OK;
  // Device layouts are compact (leading dimension = extent rounded up to 16 bytes'
  // worth of elements, so that TMA can address them).
  const size_t al = 16 / es;
  const size_t rowsA = h.transA ? h.k : h.m, colsA = h.transA ? h.m : h.k;
  const size_t dlda = align_up(rowsA ? rowsA : 1, al), dldc = align_up(h.m, al);
  // panel width: about an eighth of n, a multiple of 256 columns
  size_t np = align_up((h.n + 7) / 8, 256);
  if (np > h.n) np = h.n;
  const size_t panels = (h.n + np - 1) / np;
  const size_t dldb = h.transB ? align_up(np, al) : align_up(h.k ? h.k : 1, al);
  const size_t colsBp = h.transB ? h.k : np;  // columns of a device B panel
  const size_t a_bytes = align_up(dlda * colsA * es, 1024);
  const size_t b_bytes = align_up(dldb * (colsBp ? colsBp : 1) * es, 1024);
  const size_t c_bytes = align_up(dldc * np * es, 1024);
  HostPipe& hp = g_pipe[dev];
  int rc = pipe_setup(hp, a_bytes + 2 * b_bytes + 2 * c_bytes);
  if (rc) return rc;
  char* dA = static_cast<char*>(hp.buf);
  char* dB[2] = {dA + a_bytes, dA + a_bytes + b_bytes};
  char* dC[2] = {dA + a_bytes + 2 * b_bytes, dA + a_bytes + 2 * b_bytes + c_bytes};
  const bool use_c = dtype == MMBO_DTYPE_F64 ? beta64 != 0.0 : h.beta != 0.f;
  cudaError_t e;
  if (h.k > 0 && sharded_a && sharded_a->n_gpus > 1) {
    rc = stage_a_sharded(*sharded_a, hp, h, es, dA, dlda, rowsA, colsA);
    if (rc) { cudaDeviceSynchronize(); return rc; }
  } else {
    if (h.k > 0) {
      e = cudaMemcpy2DAsync(dA, dlda * es, h.A, h.lda * es, rowsA * es, colsA, cudaMemcpyHostToDevice, hp.s_in);
      if (e != cudaSuccess) return (int)e;
    }
    cudaEventRecord(hp.ev_a, hp.s_in);
    cudaStreamWaitEvent(hp.s_mm, hp.ev_a, 0);
  }
  for (size_t j = 0; j < panels; ++j) {
    const int b = (int)(j & 1);
    const size_t j0 = j * np, w = (j0 + np <= h.n) ? np : h.n - j0;
    if (j >= 2) {
      cudaStreamWaitEvent(hp.s_in, hp.ev_mm[b], 0);   // B buffer: its GEMM has run
      cudaStreamWaitEvent(hp.s_in, hp.ev_out[b], 0);  // C buffer: its result has left
    }
    if (h.k > 0) {
      const char* src = static_cast<const char*>(h.B) + (h.transB ? j0 : j0 * h.ldb) * es;
      if (h.transB) e = cudaMemcpy2DAsync(dB[b], dldb * es, src, h.ldb * es, w * es, h.k, cudaMemcpyHostToDevice, hp.s_in);
      else e = cudaMemcpy2DAsync(dB[b], dldb * es, src, h.ldb * es, h.k * es, w, cudaMemcpyHostToDevice, hp.s_in);
      if (e != cudaSuccess) return (int)e;
    }
    char* hCj = static_cast<char*>(h.C) + j0 * h.ldc * es;
    if (use_c) {
      e = cudaMemcpy2DAsync(dC[b], dldc * es, hCj, h.ldc * es, h.m * es, w, cudaMemcpyHostToDevice, hp.s_in);
      if (e != cudaSuccess) return (int)e;
    }
    cudaEventRecord(hp.ev_in[b], hp.s_in);
    cudaStreamWaitEvent(hp.s_mm, hp.ev_in[b], 0);
    if (j >= 2 && !use_c) cudaStreamWaitEvent(hp.s_mm, hp.ev_out[b], 0);
    GemmArgs g = h;
    g.n = w; g.A = dA; g.lda = dlda; g.B = dB[b]; g.ldb = dldb; g.C = dC[b]; g.ldc = dldc;
    int id = kernelId;
    if (dtype == MMBO_DTYPE_F64) {
      if (id == MMBO_KERNEL_AUTO) {
        id = tune_lookup(MMBO_DTYPE_F64, g);
        if (id < 0) id = select_f64(g);
      }
      rc = run_f64(g, alpha64, beta64, id, hp.s_mm);
    } else if (dtype == MMBO_DTYPE_F32) {
      if (id == MMBO_KERNEL_AUTO) id = select_f32_fitting(g);
      rc = run_f32(g, id, hp.s_mm);
    } else {
      if (id == MMBO_KERNEL_AUTO) id = select_f16(g);
      rc = run_f16(g, id, hp.s_mm);
    }
    if (rc) { cudaDeviceSynchronize(); return rc; }
    cudaEventRecord(hp.ev_mm[b], hp.s_mm);
    cudaStreamWaitEvent(hp.s_out, hp.ev_mm[b], 0);
    e = cudaMemcpy2DAsync(hCj, h.ldc * es, dC[b], dldc * es, h.m * es, w, cudaMemcpyDeviceToHost, hp.s_out);
    if (e != cudaSuccess) return (int)e;
    cudaEventRecord(hp.ev_out[b], hp.s_out);
  }
  // the caller's buffers hold the result when this returns
  if ((e = cudaStreamSynchronize(hp.s_out)) != cudaSuccess) return (int)e;
  if ((e = cudaStreamSynchronize(hp.s_mm)) != cudaSuccess) return (int)e;
  if ((e = cudaStreamSynchronize(hp.s_cc)) != cudaSuccess) return (int)e;
  return (int)cudaStreamSynchronize(hp.s_in);
}

}  // namespace mmbo

// ====================================================================== C ABI =========
using namespace mmbo;

extern "C" {

int mmbo_gemm_f32(int transA, int transB, size_t m, size_t n, size_t k, const float* alpha,
                  const float* A, size_t lda, const float* B, size_t ldb, const float* beta, float* C,
                  size_t ldc, int kernelId, void* stream) {
  MMBO_API_LOCK();
  GemmArgs g{transA, transB, m, n, k, A, B, C, lda, ldb, ldc, 0.f, 0.f};
  int rc = validate(g, alpha, beta);
  if (rc) return rc;
  g.alpha = *alpha;
  g.beta = *beta;
  if (kernelId != MMBO_KERNEL_AUTO && (kernelId < 0 || kernelId >= kNumF32)) return MMBO_ERR_BAD_KERNEL_ID;
  const int id = kernelId == MMBO_KERNEL_AUTO ? select_f32_fitting(g) : kernelId;
  return run_f32(g, id, static_cast<cudaStream_t>(stream));
}

int mmbo_gemm_f16(int transA, int transB, size_t m, size_t n, size_t k, const float* alpha, const void* A,
                  size_t lda, const void* B, size_t ldb, const float* beta, void* C, size_t ldc,
                  int kernelId, void* stream) {
  MMBO_API_LOCK();
  GemmArgs g{transA, transB, m, n, k, A, B, C, lda, ldb, ldc, 0.f, 0.f};
  int rc = validate(g, alpha, beta);
  if (rc) return rc;
  g.alpha = *alpha;
  g.beta = *beta;
  if (kernelId != MMBO_KERNEL_AUTO && (kernelId < 0 || kernelId >= kNumF16)) return MMBO_ERR_BAD_KERNEL_ID;
  const int id = kernelId == MMBO_KERNEL_AUTO ? select_f16(g) : kernelId;
  return run_f16(g, id, static_cast<cudaStream_t>(stream));
}

int mmbo_gemm_f16_bcast(int transA, int transB, size_t m, size_t n, size_t k, const float* alpha, const void* A,
                        size_t lda, const void* B, size_t ldb, const float* beta, void* C, size_t ldc,
                        void* const* C_peers, int npeers, int kernelId, void* stream) {
  MMBO_API_LOCK();
  GemmArgs g{transA, transB, m, n, k, A, B, C, lda, ldb, ldc, 0.f, 0.f};
  int rc = validate(g, alpha, beta);
  if (rc) return rc;
  g.alpha = *alpha;
  g.beta = *beta;
  if (npeers < 0 || npeers > kMaxPeerCopies) return MMBO_ERR_BAD_DIM;
  if (npeers > 0 && !C_peers) return MMBO_ERR_NULL_POINTER;
  if (kernelId != MMBO_KERNEL_AUTO && (kernelId < 1 || kernelId >= kNumF16)) return MMBO_ERR_BAD_KERNEL_ID;
  if (g.m == 0 || g.n == 0) return MMBO_OK;
  // only the tensor-core kernels with the TMA epilogue can store to further destinations
  if (g.k == 0 || !hgemm_tma_ok(g) || !aligned16(g.C) || g.ldc % 8 != 0 || g.m % 8 != 0) return MMBO_ERR_KERNEL_UNSUITABLE;
  int id = kernelId == MMBO_KERNEL_AUTO ? select_f16(g) : kernelId;
  if (id == 0) id = 2;  // the smallest tensor-core tile instead of the one-thread-per-element kernel
  g.peers = C_peers;
  g.npeers = npeers;
  return run_f16(g, id, static_cast<cudaStream_t>(stream));
}

int mmbo_gemm_f16_mcast(int transA, int transB, size_t m, size_t n, size_t k, const float* alpha, const void* A,
                        size_t lda, const void* B, size_t ldb, const float* beta, void* C, size_t ldc,
                        void* C_multicast, int kernelId, void* stream) {
  MMBO_API_LOCK();
  GemmArgs g{transA, transB, m, n, k, A, B, C, lda, ldb, ldc, 0.f, 0.f};
  int rc = validate(g, alpha, beta);
  if (rc) return rc;
  g.alpha = *alpha;
  g.beta = *beta;
  if (!C_multicast) return MMBO_ERR_NULL_POINTER;
  if (kernelId != MMBO_KERNEL_AUTO && (kernelId < 1 || kernelId >= kNumF16)) return MMBO_ERR_BAD_KERNEL_ID;
  if (g.m == 0 || g.n == 0) return MMBO_OK;
  // only the tensor-core kernels' staged epilogue writes whole 16-byte column pieces
  if (g.k == 0 || !hgemm_tma_ok(g) || !aligned16(g.C) || !aligned16(C_multicast) || g.ldc % 8 != 0 || g.m % 8 != 0)
    return MMBO_ERR_KERNEL_UNSUITABLE;
  int id = kernelId == MMBO_KERNEL_AUTO ? select_f16(g) : kernelId;
  if (id == 0) id = 2;
  g.c_multicast = C_multicast;
  return run_f16(g, id, static_cast<cudaStream_t>(stream));
}

// Checks shared by the multi-GPU entry points; on success (*col0, *ncols) is this rank's block.
static int shard_check(int nGpus, int rank, void* comm, bool need_comm, size_t n, size_t* col0, size_t* ncols) {
  if (nGpus <= 0 || nGpus > 64 || rank < 0 || rank >= nGpus) return MMBO_ERR_BAD_SHARD;
  if (need_comm && nGpus > 1) {
    if (!comm) return MMBO_ERR_NULL_POINTER;
    NcclApi& nc = nccl_api();
    if (!nc.ok()) return MMBO_ERR_NO_NCCL;
    int cnt = 0, me = -1;
    if (nc.comm_count(comm, &cnt) || nc.comm_user_rank(comm, &me)) return MMBO_ERR_NCCL;
    if (cnt != nGpus || me != rank) return MMBO_ERR_BAD_SHARD;  // the communicator is not the one described
  }
  return mmbo_shard_columns(n, nGpus, rank, 256, col0, ncols);
}

int mmbo_gemm_f16_sharded(int nGpus, int rank, void* ncclComm, int gatherC, int transA, int transB, size_t m,
                          size_t n, size_t k, const float* alpha, const void* A, size_t lda, const void* B_block,
                          size_t ldb, const float* beta, void* C, size_t ldc, int kernelId, void* stream) {
  MMBO_API_LOCK();
  size_t col0 = 0, ncols = 0;
  int rc = shard_check(nGpus, rank, ncclComm, gatherC != 0, n, &col0, &ncols);
  if (rc) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  char* c_block = C ? static_cast<char*>(C) + col0 * ldc * 2 : nullptr;
  GemmArgs g{transA, transB, m, ncols, k, A, B_block, c_block, lda, ldb, ldc, 0.f, 0.f};
  if ((rc = validate(g, alpha, beta))) return rc;
  g.alpha = *alpha;
  g.beta = *beta;
  if (kernelId != MMBO_KERNEL_AUTO && (kernelId < 0 || kernelId >= kNumF16)) return MMBO_ERR_BAD_KERNEL_ID;
  if (gatherC && nGpus > 1 && ldc != m) return MMBO_ERR_BAD_SHARD;  // column blocks must be contiguous to be exchanged
  if (m == 0 || n == 0) return MMBO_OK;
  if (ncols > 0) {
    const int id = kernelId == MMBO_KERNEL_AUTO ? select_f16(g) : kernelId;
    if ((rc = run_f16(g, id, st))) return rc;
  }
  if (!gatherC || nGpus == 1) return MMBO_OK;
  NcclApi& nc = nccl_api();
  int nrc = 0;
  if (n % ((size_t)nGpus * 256) == 0) {  // equal blocks: one all-gather in place
    nrc = nc.all_gather(c_block, C, m * ncols, kNcclFloat16, ncclComm, st);
  } else {
    nrc = nc.group_start();
    for (int r = 0; !nrc && r < nGpus; ++r) {
      size_t r0 = 0, rn = 0;
      mmbo_shard_columns(n, nGpus, r, 256, &r0, &rn);
      if (rn == 0) continue;
      char* piece = static_cast<char*>(C) + r0 * ldc * 2;
      nrc = nc.broadcast(piece, piece, m * rn, kNcclFloat16, r, ncclComm, st);
    }
    const int end = nc.group_end();
    if (!nrc) nrc = end;
  }
  return nrc ? MMBO_ERR_NCCL : MMBO_OK;
}

int mmbo_gemm_f16_sharded_host(int nGpus, int rank, void* ncclComm, int transA, int transB, size_t m, size_t n,
                               size_t k, const float* alpha, const void* A, size_t lda, const void* B_block,
                               size_t ldb, const float* beta, void* C_block, size_t ldc, int kernelId) {
  MMBO_API_LOCK();
  size_t col0 = 0, ncols = 0;
  int rc = shard_check(nGpus, rank, ncclComm, true, n, &col0, &ncols);
  if (rc) return rc;
  // Every rank takes part in the exchange of A, so every rank must own columns: the same answer on all ranks.
  if (m != 0 && n != 0 && (n + 255) / 256 < (size_t)nGpus) return MMBO_ERR_BAD_SHARD;
  GemmArgs g{transA, transB, m, ncols, k, A, B_block, C_block, lda, ldb, ldc, 0.f, 0.f};
  if ((rc = validate(g, alpha, beta))) return rc;
  g.alpha = *alpha;
  g.beta = *beta;
  if (kernelId != MMBO_KERNEL_AUTO && (kernelId < 0 || kernelId >= kNumF16)) return MMBO_ERR_BAD_KERNEL_ID;
  if (m == 0 || n == 0) return MMBO_OK;
  const ShardedA sa{nGpus, rank, ncclComm};
  return gemm_host(MMBO_DTYPE_F16, g, kernelId, 0.0, 0.0, &sa);
}

int mmbo_gemm_f32_host(int transA, int transB, size_t m, size_t n, size_t k, const float* alpha, const float* A,
                       size_t lda, const float* B, size_t ldb, const float* beta, float* C, size_t ldc,
                       int kernelId) {
  MMBO_API_LOCK();
  GemmArgs g{transA, transB, m, n, k, A, B, C, lda, ldb, ldc, 0.f, 0.f};
  int rc = validate(g, alpha, beta);
  if (rc) return rc;
  g.alpha = *alpha;
  g.beta = *beta;
  if (kernelId != MMBO_KERNEL_AUTO && (kernelId < 0 || kernelId >= kNumF32)) return MMBO_ERR_BAD_KERNEL_ID;
  return gemm_host(MMBO_DTYPE_F32, g, kernelId);
}

int mmbo_gemm_f16_host(int transA, int transB, size_t m, size_t n, size_t k, const float* alpha, const void* A,
                       size_t lda, const void* B, size_t ldb, const float* beta, void* C, size_t ldc,
                       int kernelId) {
  MMBO_API_LOCK();
  GemmArgs g{transA, transB, m, n, k, A, B, C, lda, ldb, ldc, 0.f, 0.f};
  int rc = validate(g, alpha, beta);
  if (rc) return rc;
  g.alpha = *alpha;
  g.beta = *beta;
  if (kernelId != MMBO_KERNEL_AUTO && (kernelId < 0 || kernelId >= kNumF16)) return MMBO_ERR_BAD_KERNEL_ID;
  return gemm_host(MMBO_DTYPE_F16, g, kernelId);
}

int mmbo_gemm_f64(int transA, int transB, size_t m, size_t n, size_t k, const double* alpha, const double* A,
                  size_t lda, const double* B, size_t ldb, const double* beta, double* C, size_t ldc,
                  int kernelId, void* stream) {
  MMBO_API_LOCK();
  GemmArgs g{transA, transB, m, n, k, A, B, C, lda, ldb, ldc, 0.f, 0.f};
  int rc = validate(g, reinterpret_cast<const float*>(alpha), reinterpret_cast<const float*>(beta));
  if (rc) return rc;
  if (kernelId != MMBO_KERNEL_AUTO && (kernelId < 0 || kernelId >= kNumF64)) return MMBO_ERR_BAD_KERNEL_ID;
  int id = kernelId;
  if (id == MMBO_KERNEL_AUTO) {
    id = tune_lookup(MMBO_DTYPE_F64, g);
    if (id < 0) id = select_f64(g);
  }
  return run_f64(g, *alpha, *beta, id, static_cast<cudaStream_t>(stream));
}

int mmbo_gemm_f64_host(int transA, int transB, size_t m, size_t n, size_t k, const double* alpha, const double* A,
                       size_t lda, const double* B, size_t ldb, const double* beta, double* C, size_t ldc,
                       int kernelId) {
  MMBO_API_LOCK();
  GemmArgs g{transA, transB, m, n, k, A, B, C, lda, ldb, ldc, 0.f, 0.f};
  int rc = validate(g, reinterpret_cast<const float*>(alpha), reinterpret_cast<const float*>(beta));
  if (rc) return rc;
  if (kernelId != MMBO_KERNEL_AUTO && (kernelId < 0 || kernelId >= kNumF64)) return MMBO_ERR_BAD_KERNEL_ID;
  return gemm_host(MMBO_DTYPE_F64, g, kernelId, *alpha, *beta);
}

// One launch for the whole batch where the chosen kernel can address it (the problem index is a
// coordinate of its tile walk or the third grid dimension); otherwise one call per problem.
static bool batch_in_one_launch(int dtype, int id, const GemmArgs& g) {
  if (g.batch <= 1) return true;
  if (g.batch > 65535) return false;
  if (g.k == 0 || id == 0) return true;  // grid z, any strides
  if (dtype == MMBO_DTYPE_F16)  // tensor maps over the caller's operands: strides in whole 16-byte units
    return hgemm_tma_ok(g) && batch_stride_ok(g.batch, g.sA, 2) && batch_stride_ok(g.batch, g.sB, 2);
  if (dtype == MMBO_DTYPE_F32) return id != 6;  // ids 1, 2: grid z; 3-5: the split pass reads any strides
  return true;                                  // fp64: grid z, or pointer offsets where TMA cannot take the stride
}

int mmbo_gemm_strided_batched(int dtype, int transA, int transB, size_t m, size_t n, size_t k, const void* alpha,
                              const void* A, size_t lda, size_t strideA, const void* B, size_t ldb, size_t strideB,
                              const void* beta, void* C, size_t ldc, size_t strideC, size_t batch, int kernelId,
                              void* stream) {
  MMBO_API_LOCK();
  if (dtype != MMBO_DTYPE_F16 && dtype != MMBO_DTYPE_F32 && dtype != MMBO_DTYPE_F64) return MMBO_ERR_BAD_DTYPE;
  GemmArgs g{transA, transB, m, n, k, A, B, C, lda, ldb, ldc, 0.f, 0.f};
  int rc = validate(g, static_cast<const float*>(alpha), static_cast<const float*>(beta));
  if (rc) return rc;
  int count = 0;
  rows_of(dtype, &count);
  if (kernelId != MMBO_KERNEL_AUTO && (kernelId < 0 || kernelId >= count)) return MMBO_ERR_BAD_KERNEL_ID;
  if (batch == 0 || m == 0 || n == 0) return MMBO_OK;
  double alpha64 = 0.0, beta64 = 0.0;
  if (dtype == MMBO_DTYPE_F64) {
    alpha64 = *static_cast<const double*>(alpha);
    beta64 = *static_cast<const double*>(beta);
  } else {
    g.alpha = *static_cast<const float*>(alpha);
    g.beta = *static_cast<const float*>(beta);
  }
  g.batch = batch; g.sA = strideA; g.sB = strideB; g.sC = strideC;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int id = kernelId;
  if (id == MMBO_KERNEL_AUTO) {
    if (dtype == MMBO_DTYPE_F16) id = select_f16(g);
    else if (dtype == MMBO_DTYPE_F32) id = select_f32_fitting(g);
    else {
      id = g.k == 0 ? 0 : tune_lookup(MMBO_DTYPE_F64, g);
      if (id < 0) id = select_f64(g);
    }
  }
  if (batch_in_one_launch(dtype, id, g)) {
    if (dtype == MMBO_DTYPE_F16) rc = run_f16(g, id, st);
    else if (dtype == MMBO_DTYPE_F32) rc = run_f32(g, id, st);
    else rc = run_f64(g, alpha64, beta64, id, st);
    // a stride the tensor maps refuse (the driver has the last word): one call per problem instead
    if (rc != MMBO_ERR_TENSOR_MAP) return rc;
  }
  const size_t es = dtype == MMBO_DTYPE_F16 ? 2 : dtype == MMBO_DTYPE_F32 ? 4 : 8;
  GemmArgs one = g;
  one.batch = 1; one.sA = one.sB = one.sC = 0;
  for (size_t b = 0; b < batch; ++b) {
    one.A = static_cast<const char*>(A) + (A ? b * strideA * es : 0);
    one.B = static_cast<const char*>(B) + (B ? b * strideB * es : 0);
    one.C = static_cast<char*>(C) + b * strideC * es;
    if (dtype == MMBO_DTYPE_F16) rc = run_f16(one, id, st);
    else if (dtype == MMBO_DTYPE_F32) rc = run_f32(one, id, st);
    else rc = run_f64(one, alpha64, beta64, id, st);
    if (rc) return rc;
  }
  return MMBO_OK;
}

unsigned long long mmbo_launch_count(void) {
  MMBO_API_LOCK();
  return g_launch_count;
}

int mmbo_last_kernel(int dtype) {
  MMBO_API_LOCK();
  if (dtype != MMBO_DTYPE_F32 && dtype != MMBO_DTYPE_F16 && dtype != MMBO_DTYPE_F64) return MMBO_ERR_BAD_DTYPE;
  return g_last_kernel[dtype];
}

int mmbo_set_option(const char* name, unsigned int value) {
  MMBO_API_LOCK();
  if (!name) return MMBO_ERR_NULL_POINTER;
  Settings& s = settings();
  if (!strcmp(name, "diag")) s.diag = value;
  else if (!strcmp(name, "wgm")) s.wgm = value;
  else if (!strcmp(name, "tf32_chunk")) s.tf32_chunk = value ? value : 1;
  else if (!strcmp(name, "f32_exact")) s.f32_exact = value;
  else if (!strcmp(name, "dgemm_stage_c")) s.dgemm_stage_c = value;
  else if (!strcmp(name, "split_k")) s.split_k = value;
  else if (!strcmp(name, "pdl")) s.pdl = value;
  else return MMBO_ERR_BAD_OPTION;
  return MMBO_OK;
}

int mmbo_get_option(const char* name, unsigned int* value) {
  MMBO_API_LOCK();
  if (!name || !value) return MMBO_ERR_NULL_POINTER;
  const Settings& s = settings();
  if (!strcmp(name, "diag")) *value = s.diag;
  else if (!strcmp(name, "wgm")) *value = s.wgm;
  else if (!strcmp(name, "tf32_chunk")) *value = s.tf32_chunk;
  else if (!strcmp(name, "f32_exact")) *value = s.f32_exact;
  else if (!strcmp(name, "dgemm_stage_c")) *value = s.dgemm_stage_c;
  else if (!strcmp(name, "split_k")) *value = s.split_k;
  else if (!strcmp(name, "pdl")) *value = s.pdl;
  else return MMBO_ERR_BAD_OPTION;
  return MMBO_OK;
}

int mmbo_num_kernels(int dtype) {
  int n = 0;
  rows_of(dtype, &n);
  return n;
}

const char* mmbo_kernel_name(int dtype, int kernelId) {
  int n = 0;
  const KernelRow* r = rows_of(dtype, &n);
  if (!r || kernelId < 0 || kernelId >= n) return nullptr;
  return r[kernelId].name;
}

int mmbo_kernel_params(int dtype, int kernelId, int out[8]) {
  int n = 0;
  const KernelRow* r = rows_of(dtype, &n);
  if (!r) return MMBO_ERR_BAD_DTYPE;
  if (kernelId < 0 || kernelId >= n) return MMBO_ERR_BAD_KERNEL_ID;
  if (!out) return MMBO_ERR_NULL_POINTER;
  const KernelRow& k = r[kernelId];
  out[0] = k.mt0; out[1] = k.mt1; out[2] = k.threads; out[3] = k.depth_u;
  out[4] = k.stages; out[5] = k.cta_group; out[6] = k.wgm; out[7] = k.tensor;
  return MMBO_OK;
}

int mmbo_select_kernel(int dtype, int transA, int transB, size_t m, size_t n, size_t k, const void* A,
                       size_t lda, const void* B, size_t ldb, const void* C, size_t ldc) {
  MMBO_API_LOCK();
  GemmArgs g{transA, transB, m, n, k, A, B, const_cast<void*>(C), lda, ldb, ldc, 1.f, 1.f};  // (as for beta != 0)
  const float one = 1.f;
  int rc = validate(g, &one, &one);
  if (rc) return rc;
  if (dtype == MMBO_DTYPE_F32) return select_f32(g);
  if (dtype == MMBO_DTYPE_F16) return select_f16(g);
  if (dtype == MMBO_DTYPE_F64) {
    if (g.k == 0) return 0;
    const int tuned = tune_lookup(MMBO_DTYPE_F64, g);
    return tuned >= 0 ? tuned : select_f64(g);
  }
  return MMBO_ERR_BAD_DTYPE;
}

const char* mmbo_status_string(int status) {
  switch (status) {
    case MMBO_OK: return "ok";
    case MMBO_ERR_BAD_TRANS: return "transA/transB must be 0 or 1";
    case MMBO_ERR_BAD_DIM: return "m, n or k out of range";
    case MMBO_ERR_NULL_POINTER: return "null pointer argument";
    case MMBO_ERR_BAD_LDA: return "lda smaller than the leading extent of A";
    case MMBO_ERR_BAD_LDB: return "ldb smaller than the leading extent of B";
    case MMBO_ERR_BAD_LDC: return "ldc smaller than m";
    case MMBO_ERR_BAD_KERNEL_ID: return "kernelId outside the kernel table";
    case MMBO_ERR_KERNEL_UNSUITABLE: return "forced kernel cannot address these operands (alignment)";
    case MMBO_ERR_BAD_DTYPE: return "unknown dtype";
    case MMBO_ERR_BAD_SHARD: return "bad shard arguments";
    case MMBO_ERR_NO_DRIVER_ENTRY: return "cuTensorMapEncodeTiled unavailable";
    case MMBO_ERR_TENSOR_MAP: return "tensor map rejected by the driver";
    case MMBO_ERR_DEVICE_FAULT: return "a kernel recorded a bounded-wait time-out";
    case MMBO_ERR_TOO_LARGE: return "problem exceeds launch limits of the chosen kernel";
    case MMBO_ERR_WORKSPACE: return "the workspace lent by the caller is too small for this call";
    case MMBO_ERR_TUNING_FILE: return "tuning file missing or malformed";
    case MMBO_ERR_BAD_OPTION: return "unknown option name";
    case MMBO_ERR_NCCL: return "an NCCL call on the caller's communicator failed";
    case MMBO_ERR_NO_NCCL: return "libnccl.so.2 could not be found in the process";
    case MMBO_ERR_NOALLOC_TOO_LARGE:
      return "problem needs more scratch than the library's built-in MMBO_NOALLOC_SCRATCH_BYTES";
  }
  if (status > 0) return cudaGetErrorString(static_cast<cudaError_t>(status));
  return "unknown status";
}

void mmbo_wgm_map(uint32_t wg0, uint32_t wg1, uint32_t nwg0, uint32_t nwg1, uint32_t wgm, uint32_t* tile0,
                  uint32_t* tile1) {
  mmbo_wgm_remap(wg0, wg1, nwg0, nwg1, wgm, tile0, tile1);
}

int mmbo_shard_columns(size_t n, int nGpus, int rank, size_t align, size_t* col0, size_t* ncols) {
  if (nGpus <= 0 || rank < 0 || rank >= nGpus || !col0 || !ncols) return MMBO_ERR_BAD_SHARD;
  if (align == 0) align = 1;
  const size_t units = (n + align - 1) / align;  // column groups of `align`
  const size_t base = units / (size_t)nGpus, extra = units % (size_t)nGpus;
  const size_t r = (size_t)rank;
  const size_t u0 = r * base + (r < extra ? r : extra);
  const size_t un = base + (r < extra ? 1 : 0);
  size_t c0 = u0 * align, c1 = (u0 + un) * align;
  if (c0 > n) c0 = n;
  if (c1 > n) c1 = n;
  *col0 = c0;
  *ncols = c1 - c0;
  return MMBO_OK;
}

static int fill_common(int dtype, void* dst, size_t rows, size_t cols, size_t ld, uint64_t seed, uint32_t mat,
                       int dist, float scale, size_t row0, size_t col0, size_t total_rows, void* stream) {
  MMBO_API_LOCK();
  if (rows == 0 || cols == 0) return MMBO_OK;
  if (!dst) return MMBO_ERR_NULL_POINTER;
  if (ld < rows) return MMBO_ERR_BAD_LDC;
  const size_t total = rows * cols;
  size_t blocks = (total + 255) / 256;
  const size_t cap = (size_t)sm_count() * 32;
  if (blocks > cap) blocks = cap;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == MMBO_DTYPE_F32)
    fill_kernel<float><<<(unsigned)blocks, 256, 0, st>>>(static_cast<float*>(dst), rows, cols, ld, seed, mat,
                                                         dist, scale, row0, col0, total_rows);
  else if (dtype == MMBO_DTYPE_F64)
    fill_kernel<double><<<(unsigned)blocks, 256, 0, st>>>(static_cast<double*>(dst), rows, cols, ld, seed, mat,
                                                          dist, scale, row0, col0, total_rows);
  else
    fill_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>(static_cast<__half*>(dst), rows, cols, ld, seed,
                                                          mat, dist, scale, row0, col0, total_rows);
  return (int)cudaGetLastError();
}

int mmbo_fill_f32(float* dst, size_t rows, size_t cols, size_t ld, uint64_t seed, uint32_t mat, int dist,
                  float scale, size_t row0, size_t col0, size_t total_rows, void* stream) {
  return fill_common(MMBO_DTYPE_F32, dst, rows, cols, ld, seed, mat, dist, scale, row0, col0, total_rows, stream);
}

int mmbo_fill_f64(double* dst, size_t rows, size_t cols, size_t ld, uint64_t seed, uint32_t mat, int dist,
                  float scale, size_t row0, size_t col0, size_t total_rows, void* stream) {
  return fill_common(MMBO_DTYPE_F64, dst, rows, cols, ld, seed, mat, dist, scale, row0, col0, total_rows, stream);
}

int mmbo_fill_f16(void* dst, size_t rows, size_t cols, size_t ld, uint64_t seed, uint32_t mat, int dist,
                  float scale, size_t row0, size_t col0, size_t total_rows, void* stream) {
  return fill_common(MMBO_DTYPE_F16, dst, rows, cols, ld, seed, mat, dist, scale, row0, col0, total_rows, stream);
}

int mmbo_gemm_workspace_bytes(int dtype, int kernelId, size_t m, size_t n, size_t k, size_t* bytes) {
  MMBO_API_LOCK();
  if (!bytes) return MMBO_ERR_NULL_POINTER;
  int count = 0;
  if (!rows_of(dtype, &count)) return MMBO_ERR_BAD_DTYPE;
  if (kernelId < 0 || kernelId >= count) return MMBO_ERR_BAD_KERNEL_ID;
  *bytes = 0;
  if (dtype == MMBO_DTYPE_F32 && kernelId >= 3 && kernelId <= 5 && m && n && k) *bytes = tf32_scratch(m, n, k).total;
  // fp16 tensor-core rows: worst case, both operands need an aligned copy
  if (dtype == MMBO_DTYPE_F16 && kernelId >= 1 && m && n && k)
    *bytes = align_up(align_up(m > k ? m : k, 8) * (m > k ? m : k) * 2, 1024) +
             align_up(align_up(n > k ? n : k, 8) * (n > k ? n : k) * 2, 1024);
  return MMBO_OK;
}

int mmbo_set_workspace(void* ptr, size_t bytes) {
  MMBO_API_LOCK();
  const int dev = current_device();
  if (dev < 0 || dev >= kMaxDevices) return MMBO_ERR_TOO_LARGE;
  // reject before touching any state: a refused call leaves the library as it was
  if (ptr && (reinterpret_cast<uintptr_t>(ptr) & 1023u)) return MMBO_ERR_WORKSPACE;
  Workspace& w = g_ws[dev];
  if (!w.user && w.ptr) {
    cudaError_t e = cudaFree(w.ptr);  // waits for the kernels still using it
    w.ptr = nullptr;
    w.bytes = 0;
    if (e != cudaSuccess) return (int)e;
  }
  w.ptr = ptr;
  w.bytes = ptr ? bytes : 0;
  w.user = ptr != nullptr;
  return MMBO_OK;
}

int mmbo_tuning_set(int dtype, int transA, int transB, size_t m, size_t n, size_t k, int kernelId) {
  MMBO_API_LOCK();
  if ((transA != 0 && transA != 1) || (transB != 0 && transB != 1)) return MMBO_ERR_BAD_TRANS;
  return tune_set(dtype, transA, transB, m, n, k, kernelId);
}

int mmbo_tuning_set_split(int dtype, int transA, int transB, size_t m, size_t n, size_t k, int kernelId, int split) {
  MMBO_API_LOCK();
  if ((transA != 0 && transA != 1) || (transB != 0 && transB != 1)) return MMBO_ERR_BAD_TRANS;
  return tune_set(dtype, transA, transB, m, n, k, kernelId, split);
}

int mmbo_tuning_load(const char* path) {
  MMBO_API_LOCK();
  if (!path) return MMBO_ERR_NULL_POINTER;
  return tune_load(path);
}

void mmbo_tuning_clear(void) {
  MMBO_API_LOCK();
  g_tune_count = 0;
  g_tune_env_done = true;  // an explicit clear also cancels the environment file
}

int mmbo_selftest_bounded_wait(unsigned long long limit_ns, void* stream) {
  if (limit_ns == 0 || limit_ns > 1000000000ull) return MMBO_ERR_BAD_DIM;
  bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(limit_ns);
  return (int)cudaGetLastError();
}

int mmbo_debug_trace(int enable, unsigned long long* out, size_t words) {
  MMBO_API_LOCK();
  // enable != 0: allocate and clear the trace buffer, later launches record into it;
  // enable == 0: copy up to `words` words to `out` (host) and disarm.
  if (enable) {
    if (!g_trace_buffer) {
      cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&g_trace_buffer), kTraceWords * 8);
      if (e != cudaSuccess) return (int)e;
    }
    return (int)cudaMemset(g_trace_buffer, 0, kTraceWords * 8);
  }
  if (!g_trace_buffer) return MMBO_OK;
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess && out) e = cudaMemcpy(out, g_trace_buffer, (words < kTraceWords ? words : kTraceWords) * 8, cudaMemcpyDeviceToHost);
  cudaFree(g_trace_buffer);
  g_trace_buffer = nullptr;
  return (int)e;
}

int mmbo_device_status(unsigned int* status) {
  MMBO_API_LOCK();
  if (!status) return MMBO_ERR_NULL_POINTER;
  unsigned int v = 0;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return (int)e;
  e = cudaMemcpyFromSymbol(&v, g_mmbo_device_status, sizeof v);
  if (e != cudaSuccess) return (int)e;
  if (v != 0) {
    const unsigned int zero = 0;
    e = cudaMemcpyToSymbol(g_mmbo_device_status, &zero, sizeof zero);
    if (e != cudaSuccess) return (int)e;
  }
  *status = v;
  return v ? MMBO_ERR_DEVICE_FAULT : MMBO_OK;
}

// ---------------------------------------------------------------- no-allocation SGEMM --
// Scratch for mmbo_gemm_f32_noalloc: part of the library image, so every GPU that loads
// the library carries these bytes until the process exits.  In host code the name below
// is only a handle for cudaGetSymbolAddress; the device address it resolves to (one per
// device) is what the kernels receive.
static __device__ __align__(256) unsigned char g_noalloc_scratch[MMBO_NOALLOC_SCRATCH_BYTES];
static void* g_noalloc_scratch_addr[kMaxDevices];

int mmbo_gemm_f32_noalloc(int transA, int transB, size_t m, size_t n, size_t k, const float* alpha,
                          const float* A, size_t lda, const float* B, size_t ldb, const float* beta, float* C,
                          size_t ldc, void* stream) {
  MMBO_API_LOCK();
  GemmArgs g{transA, transB, m, n, k, A, B, C, lda, ldb, ldc, 0.f, 0.f};
  int rc = validate(g, alpha, beta);
  if (rc) return rc;
  g.alpha = *alpha;
  g.beta = *beta;
  if (m == 0 || n == 0) return MMBO_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (k == 0) return launch_scale<float>(g, st);
  if (tf32_scratch(m, n, k).total > (size_t)MMBO_NOALLOC_SCRATCH_BYTES) return MMBO_ERR_NOALLOC_TOO_LARGE;
  const int dev = current_device();
  if (dev < 0 || dev >= kMaxDevices) return MMBO_ERR_TOO_LARGE;
  if (!g_noalloc_scratch_addr[dev]) {
    // once per device, with that device current: resolve the array's address there
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    g_noalloc_scratch_addr[dev] = ptr;
  }
  return run_tf32x3<128, 3, 1>(g, g_noalloc_scratch_addr[dev], wgm_of(kF32Rows[4]), st);
}

}  // extern "C"
