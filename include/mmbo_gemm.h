/*
 * mmbo_gemm.h -- C ABI of libmmbo_gemm.so, the B200 (sm_100a) GEMM library that stands
 * in for the launch surface of CSWater/GEMM_MMBO (src/gemm/gemm.h, src/gemm/driver.h,
 * src/gemm/constants.h).  Plain pointers and sizes only.
 *
 * Conventions (all entry points):
 *   - matrices are column-major; op(A) is m x k, op(B) is k x n, C is m x n;
 *       transA == 0: A is stored m x k, lda >= m      transA != 0: stored k x m, lda >= k
 *       transB == 0: B is stored k x n, ldb >= k      transB != 0: stored n x k, ldb >= n
 *     so transA = 0, transB = 1 is the reference's only layout ("NT", ldb >= n:
 *     src/gemm/benchmark.cc:26,111);
 *   - A, B, C are DEVICE pointers owned by the caller; alpha and beta are HOST pointers
 *     read during the call (src/gemm/gemm.h:31-32,76-77);
 *   - C = beta != 0 ? alpha*op(A)*op(B) + beta*C : alpha*op(A)*op(B); with beta == 0 the
 *     old contents of C are never read (src/gemm/ref/Kernels.cpp:87);
 *   - the work is queued on `stream` (a cudaStream_t; NULL = the default stream, which
 *     is what the reference uses: src/gemm/driver.h:56-59) and the call returns without
 *     waiting for it;
 *   - the return value is 0 on success, negative for a rejected argument (see
 *     mmbo_status_string), positive for a CUDA runtime error code.  Nothing is printed
 *     and the process is never terminated (the reference prints and calls exit(0):
 *     src/gemm/common.h:20-24).
 */
#ifndef MMBO_GEMM_H_
#define MMBO_GEMM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MMBO_DTYPE_F32 0
#define MMBO_DTYPE_F16 1
#define MMBO_DTYPE_F64 2

#define MMBO_KERNEL_AUTO (-1)

/* status codes */
#define MMBO_OK 0
#define MMBO_ERR_BAD_TRANS (-1)
#define MMBO_ERR_BAD_DIM (-2)
#define MMBO_ERR_NULL_POINTER (-3)
#define MMBO_ERR_BAD_LDA (-4)
#define MMBO_ERR_BAD_LDB (-5)
#define MMBO_ERR_BAD_LDC (-6)
#define MMBO_ERR_BAD_KERNEL_ID (-7)
#define MMBO_ERR_KERNEL_UNSUITABLE (-8) /* forced kernel id cannot run these operands */
#define MMBO_ERR_BAD_DTYPE (-9)
#define MMBO_ERR_BAD_SHARD (-10)
#define MMBO_ERR_NO_DRIVER_ENTRY (-11)  /* cuTensorMapEncodeTiled not available */
#define MMBO_ERR_TENSOR_MAP (-12)       /* the driver rejected a tensor map */
#define MMBO_ERR_DEVICE_FAULT (-13)     /* a kernel recorded a bounded-wait time-out */
#define MMBO_ERR_TOO_LARGE (-14)
#define MMBO_ERR_WORKSPACE (-15)        /* lent workspace too small or misaligned */
#define MMBO_ERR_TUNING_FILE (-17)      /* tuning file missing or malformed */
#define MMBO_ERR_NOALLOC_TOO_LARGE (-16) /* mmbo_gemm_f32_noalloc: scratch need exceeds the built-in array */
#define MMBO_ERR_BAD_OPTION (-18)       /* mmbo_set_option / mmbo_get_option: unknown name */
#define MMBO_ERR_NCCL (-19)             /* an NCCL call on the caller's communicator failed */
#define MMBO_ERR_NO_NCCL (-20)          /* no libnccl.so.2 in the process or on the loader path */

/* SGEMM, fp32 storage and arithmetic.  Replaces dgemm_NT / naive_dgemm
 * (src/gemm/gemm.h:47-48, :4-5) for dtype fp32; kernelId indexes the fp32 kernel table
 * (mmbo_kernel_name) the way the reference's kernelId indexes constants.h:49-135, and
 * MMBO_KERNEL_AUTO lets the library choose. */
int mmbo_gemm_f32(int transA, int transB, size_t m, size_t n, size_t k, const float* alpha,
                  const float* A, size_t lda, const float* B, size_t ldb, const float* beta,
                  float* C, size_t ldc, int kernelId, void* stream);

/* HGEMM: IEEE binary16 storage for A, B, C (passed as void*), fp32 accumulation and fp32
 * alpha/beta.  Same role as above for dtype fp16 (src/gemm/gemm.h:47-48). */
int mmbo_gemm_f16(int transA, int transB, size_t m, size_t n, size_t k, const float* alpha,
                  const void* A, size_t lda, const void* B, size_t ldb, const float* beta,
                  void* C, size_t ldc, int kernelId, void* stream);

/* HGEMM whose result is written to C and, chunk by chunk from the same epilogue, to `npeers`
 * (0..7) further copies of the same window of C: C_peers[i] is the address of C(0,0) in copy i,
 * same ldc.  Meant for copies that live on other GPUs of the node (peer mappings): a GEMM
 * sharded by column blocks then leaves the assembled C on every GPU without a separate
 * all-gather.  With beta != 0 the old values are read from C only.  Needs the tensor-core
 * kernels with the TMA epilogue: 16-byte aligned A, B, C and copies, lda, ldb, ldc multiples
 * of 8, m a multiple of 8, k > 0; otherwise MMBO_ERR_KERNEL_UNSUITABLE.  The copies are complete when
 * the stream reaches the end of the call; telling the other GPUs so is the caller's
 * business (a barrier across ranks).  No counterpart in the reference, which drives one GPU
 * (device index fixed: src/gemm/benchmark.cc:54). */
int mmbo_gemm_f16_bcast(int transA, int transB, size_t m, size_t n, size_t k, const float* alpha,
                        const void* A, size_t lda, const void* B, size_t ldb, const float* beta,
                        void* C, size_t ldc, void* const* C_peers, int npeers, int kernelId,
                        void* stream);

/* The same exchange through one multicast address.  C_multicast is the address of C(0,0) in a
 * multicast mapping of the buffers that hold C on the GPUs of the node (NVLink multicast object:
 * cuMulticastCreate / cuMulticastBindMem, or the multicast pointer of a symmetric-memory
 * allocation); C is this GPU's own, ordinary address of the same window.  The epilogue writes
 * every finished piece once, with multimem.st, to C_multicast -- the switch delivers it to every
 * bound GPU, this one included -- so the result leaves this GPU once instead of once per peer.
 * With beta != 0 the old values are read from C.  Same requirements as mmbo_gemm_f16_bcast.
 * The process must keep the multicast mapping alive until the stream has passed the call.  No
 * counterpart in the reference (one GPU: src/gemm/benchmark.cc:54). */
int mmbo_gemm_f16_mcast(int transA, int transB, size_t m, size_t n, size_t k, const float* alpha,
                        const void* A, size_t lda, const void* B, size_t ldb, const float* beta,
                        void* C, size_t ldc, void* C_multicast, int kernelId, void* stream);

/* One GEMM sharded over the GPUs of a node by column blocks of op(B) and C (new capability: the
 * reference drives one GPU, device index fixed, src/gemm/benchmark.cc:54).  One process per GPU;
 * every rank calls with the same m, n, k (the WHOLE problem) and its own rank.  Rank r owns the
 * columns mmbo_shard_columns(n, nGpus, r, 256) gives.  A (all of it) and C (the whole m x n
 * matrix, ldc) are this GPU's; B_block is this rank's block of op(B): k x ncols (ldb >= k) for
 * transB == 0, ncols x k (ldb >= ncols) for transB != 0.  The rank computes its block of C in
 * place; there is no communication in the contraction.  gatherC != 0: afterwards the blocks are
 * exchanged with NCCL on `stream` (ncclAllGather in place for equal blocks, a group of
 * ncclBroadcast otherwise), so that every rank ends with the whole C; needs ldc == m.
 * ncclComm is the caller's ncclComm_t for these nGpus ranks (may be NULL when gatherC == 0); the
 * library looks NCCL up in the process at run time (MMBO_ERR_NO_NCCL if there is none) and checks
 * that the communicator has nGpus ranks and this rank.  Collective when gatherC != 0: every rank
 * must make the call, in the same order relative to its other NCCL calls. */
int mmbo_gemm_f16_sharded(int nGpus, int rank, void* ncclComm, int gatherC, int transA, int transB,
                          size_t m, size_t n, size_t k, const float* alpha, const void* A, size_t lda,
                          const void* B_block, size_t ldb, const float* beta, void* C, size_t ldc,
                          int kernelId, void* stream);

/* The same with operands in HOST memory, for the round trip the reference's harness makes
 * (src/gemm/benchmark.cc:57-63, src/gemm/test.cc:89).  A is the whole of A in host memory (every
 * rank sees the same contents); B_block and C_block are this rank's column blocks (C_block: m x
 * ncols, ldc).  Rank r copies only ITS share of A's stored columns to its GPU
 * (mmbo_shard_columns(columns of the stored A, nGpus, r, 8)); the shares then travel between the
 * GPUs over NVLink (ncclAllGather / grouped ncclBroadcast on an internal stream), so the host
 * bridge carries A once per node instead of once per GPU.  B and C blocks go through the same
 * overlapped panel pipeline as mmbo_gemm_f16_host.  Returns when C_block holds the result.
 * Collective: every rank of the communicator must make the call; a problem with fewer than nGpus
 * blocks of 256 columns (some rank would own nothing) is refused on every rank (MMBO_ERR_BAD_SHARD). */
int mmbo_gemm_f16_sharded_host(int nGpus, int rank, void* ncclComm, int transA, int transB, size_t m,
                               size_t n, size_t k, const float* alpha, const void* A, size_t lda,
                               const void* B_block, size_t ldb, const float* beta, void* C_block,
                               size_t ldc, int kernelId);

/* The same GEMMs on operands in HOST memory: A, B, C are host pointers (pinned memory
 * gives full copy bandwidth), everything else as above.  This is the whole round trip
 * the reference's harness performs around its kernel (device allocation, hipMemcpy in,
 * launch, hipMemcpy out: src/gemm/benchmark.cc:57-63, src/gemm/test.cc:53-66,89), done
 * inside the library with the copies of B/C column panels overlapped with the GEMM on
 * internal streams.  The call returns when C holds the result.  The library keeps the
 * device staging buffers (A plus two B and two C panels) between calls. */
int mmbo_gemm_f32_host(int transA, int transB, size_t m, size_t n, size_t k, const float* alpha,
                       const float* A, size_t lda, const float* B, size_t ldb, const float* beta,
                       float* C, size_t ldc, int kernelId);
int mmbo_gemm_f16_host(int transA, int transB, size_t m, size_t n, size_t k, const float* alpha,
                       const void* A, size_t lda, const void* B, size_t ldb, const float* beta,
                       void* C, size_t ldc, int kernelId);

/* DGEMM, binary64 storage and arithmetic: the reference's own data type.  Literal
 * replacement for dgemm_NT (transA = 0, transB = 1) and naive_dgemm
 * (src/gemm/gemm.h:47-48, :4-5), which take double* alpha/beta. */
int mmbo_gemm_f64(int transA, int transB, size_t m, size_t n, size_t k, const double* alpha,
                  const double* A, size_t lda, const double* B, size_t ldb, const double* beta,
                  double* C, size_t ldc, int kernelId, void* stream);
/* The same with A, B and C in host memory, as mmbo_gemm_f32_host: the whole of what the
 * reference's benchmark does around dgemm_NT (hipMalloc, hipMemcpy in, launch, hipMemcpy
 * out: src/gemm/benchmark.cc:57-63,72-88) in one call. */
int mmbo_gemm_f64_host(int transA, int transB, size_t m, size_t n, size_t k, const double* alpha,
                       const double* A, size_t lda, const double* B, size_t ldb, const double* beta,
                       double* C, size_t ldc, int kernelId);

/* Strided-batched GEMM: problem b of `batch` uses A + b*strideA, B + b*strideB,
 * C + b*strideC (strides in elements).  The reference's Tensile argument block already
 * carries a batch index and these strides (strideC2K / strideA2K / strideB2K and sizeK,
 * src/gemm/gemm.h:62-69,88-92) with sizeK fixed to 1, and its kernel takes the problem
 * index from the third grid dimension (src/gemm/ref/Kernels.cpp:254).  alpha and beta
 * point to float for f16/f32 and to double for f64.  The whole batch is ONE launch: the
 * problem index is a coordinate of the persistent tile walk (tensor-core kernels, 3-D
 * tensor maps whose outermost dimension is the batch) or the third grid dimension (the
 * other kernels).  Falls back to one call per problem only where a kernel cannot address
 * the batch: fp16 operands that need realigning or strides that are not whole 16-byte
 * units, fp32 row 6, more than 65535 problems. */
int mmbo_gemm_strided_batched(int dtype, int transA, int transB, size_t m, size_t n, size_t k,
                              const void* alpha, const void* A, size_t lda, size_t strideA,
                              const void* B, size_t ldb, size_t strideB, const void* beta, void* C,
                              size_t ldc, size_t strideC, size_t batch, int kernelId, void* stream);

/* Kernel table -- the counterpart of naive_kernels / kernels / *_kernel_parameters in
 * src/gemm/constants.h:4-135.  out[8] = {MT0 (tile along m), MT1 (tile along n), threads,
 * DepthU (k per stage), stages, ctaGroup, wgm, usesTensorCores}. */
int mmbo_num_kernels(int dtype);
const char* mmbo_kernel_name(int dtype, int kernelId);
int mmbo_kernel_params(int dtype, int kernelId, int out[8]);
/* Kernel id that MMBO_KERNEL_AUTO resolves to for these operands (same checks as the
 * gemm call; A, B, C may be any pointers with the alignment of the real ones).  The answer is the
 * one for beta != 0; with beta == 0 a call may take the fp16 row with more operand stages instead
 * of the one with a second set of staging buffers for old C. */
int mmbo_select_kernel(int dtype, int transA, int transB, size_t m, size_t n, size_t k,
                       const void* A, size_t lda, const void* B, size_t ldb, const void* C,
                       size_t ldc);

/* Tuning table: exact-size overrides of automatic selection, the counterpart of the
 * reference's Tensile library logic (src/gemm/ref/vega20_Cijk_Ailk_Bjlk_DB.yaml:929-1177).
 * A row says "for this dtype, transpose mode and (m, n, k) use this kernel id".
 * mmbo_tuning_load reads rows from a text file (one row per line:
 * "<f16|f32|f64> <NN|NT|TN|TT> m n k kernelId", '#' comments); the file named by the
 * environment variable MMBO_TUNING_FILE is loaded on the first automatic selection.
 * gemm_mmbo_b200/autotune.py measures every kernel on a list of sizes and writes such a
 * file (the brute-force sweep of src/gemm/benchmark.cc:92-106, persisted). */
int mmbo_tuning_set(int dtype, int transA, int transB, size_t m, size_t n, size_t k, int kernelId);
/* The same with a split mode for the contraction of that problem (0 decided per call, 1 never, 2
 * always: stream-K in the rows that have it -- fp64 rows 3 and 4, fp32 row 6), the counterpart of a
 * tuned GlobalSplitU value (src/gemm/ref/vega20_Cijk_Ailk_Bjlk_DB.yaml:69-71).  In a tuning file the
 * split mode is an optional seventh field of a row.  The option "split_k", when non-zero, wins. */
int mmbo_tuning_set_split(int dtype, int transA, int transB, size_t m, size_t n, size_t k, int kernelId,
                          int split);
int mmbo_tuning_load(const char* path);
void mmbo_tuning_clear(void);

const char* mmbo_status_string(int status);

/* Switches for experiments and diagnosis, by name:
 *   "diag"          diagnostic kernels whose results are wrong by design (bit 0: no C store,
 *                   bit 1: no accumulator drain) -- the counterpart of the reference's
 *                   src/gemm/assembly/test_main_loop.s and error_kernel_000.s;
 *   "wgm"           work-group-mapping width for every kernel (0 = each table row's own;
 *                   the reference fixes 8: src/gemm/ref/Kernels.cpp:209);
 *   "tf32_chunk"    stages per tensor-memory accumulation chain of the 3xTF32 kernels;
 *   "f32_exact"     non-zero: automatic fp32 selection never takes a split-precision row,
 *                   tuned rows included;
 *   "dgemm_stage_c" 64-row fp64 tiles stage the old C through shared memory (default 1);
 *   "split_k"       0 automatic, 1 never split the contraction, n > 1 force n slices;
 *   "pdl"           non-zero (default): the persistent fp16 tensor-core kernels are launched with
 *                   programmatic stream serialization, so that their set-up overlaps the end of the
 *                   kernel before them in the stream; they wait for that kernel to complete before
 *                   they touch global memory, so results and stream order are unchanged.
 * Initial values come from the environment variables MMBO_DIAG, MMBO_WGM, MMBO_TF32_CHUNK,
 * MMBO_F32_EXACT, MMBO_DGEMM_STAGE_C, MMBO_SPLIT_K, MMBO_PDL, which are read once, when the first
 * call needs a setting; later changes of the environment have no effect.  (The reference has
 * compile-time #defines only: src/gemm/benchmark.cc:7-14.) */
int mmbo_set_option(const char* name, unsigned int value);
int mmbo_get_option(const char* name, unsigned int* value);

/* Number of kernel launches this library has queued since it was loaded (GEMM, split and
 * scale kernels; not the operand generator).  For tests and benchmarks that state how many
 * launches a call costs (the reference launches exactly one kernel per call:
 * src/gemm/driver.h:56-59). */
unsigned long long mmbo_launch_count(void);

/* Table row that the most recent GEMM call of `dtype` in this process ran (the row an automatic
 * selection resolved to -- it depends on beta, which mmbo_select_kernel does not see), -1 before
 * the first call; MMBO_ERR_BAD_DTYPE for an unknown dtype.  The reference prints the kernel it
 * picked from its own table: src/gemm/benchmark.cc:92-106. */
int mmbo_last_kernel(int dtype);

/* Tile rasterisation used by the kernels (the reference's work-group mapping,
 * src/gemm/ref/Kernels.cpp:209-236), exposed for host-side checks. */
void mmbo_wgm_map(uint32_t wg0, uint32_t wg1, uint32_t nwg0, uint32_t nwg1, uint32_t wgm,
                  uint32_t* tile0, uint32_t* tile1);

/* Column-block partition of an n-column B/C among nGpus ranks: rank r owns columns
 * [*col0, *col0 + *ncols).  Blocks are multiples of `align` columns except the last. */
int mmbo_shard_columns(size_t n, int nGpus, int rank, size_t align, size_t* col0, size_t* ncols);

/* Seeded operand generator on the device (replaces the rand()/RAND_MAX host loops of
 * src/gemm/benchmark.cc:44-52): fills the rows x cols window of a column-major array with
 * the values of logical elements (row0 + i, col0 + j) of matrix `mat` (mmbo_rng.h). */
int mmbo_fill_f32(float* dst, size_t rows, size_t cols, size_t ld, uint64_t seed, uint32_t mat,
                  int dist, float scale, size_t row0, size_t col0, size_t total_rows, void* stream);
int mmbo_fill_f16(void* dst, size_t rows, size_t cols, size_t ld, uint64_t seed, uint32_t mat,
                  int dist, float scale, size_t row0, size_t col0, size_t total_rows, void* stream);
int mmbo_fill_f64(double* dst, size_t rows, size_t cols, size_t ld, uint64_t seed, uint32_t mat,
                  int dist, float scale, size_t row0, size_t col0, size_t total_rows, void* stream);

/* Scratch memory.  Some kernels repack their operands into scratch memory (today: the
 * 3xTF32 SGEMM rows of the fp32 table).  By default the library keeps one buffer per
 * device and grows it with cudaMalloc on demand (the reference allocates nothing: its
 * kernels need no scratch).  mmbo_gemm_workspace_bytes tells how much a call with a given
 * kernel id needs (0 for kernels without scratch); mmbo_set_workspace lends the library a
 * caller-owned, 1024-byte aligned device buffer for the current device (ptr = NULL hands
 * control back to the library).  With a lent buffer the library never allocates and a
 * call that needs more returns MMBO_ERR_WORKSPACE.  Calls that use the same scratch
 * buffer must not overlap on the GPU. */
int mmbo_gemm_workspace_bytes(int dtype, int kernelId, size_t m, size_t n, size_t k, size_t* bytes);
int mmbo_set_workspace(void* ptr, size_t bytes);

/* SGEMM that allocates nothing.  (No counterpart in the reference, whose kernels use no
 * scratch memory.)
 *
 * Who needs it: code that must not call cudaMalloc at the moment it needs a GEMM --
 * a real-time or latency-critical loop where an allocation (which can synchronise the
 * whole device) is unacceptable, a plugin running inside a host application that owns
 * all device memory and forbids its guests to allocate, or a process whose memory pool
 * is already exhausted.  For them the split-precision tensor-core SGEMM (row 4 of the
 * fp32 table: every operand is split into tf32 hi/lo parts and repacked before the GEMM)
 * is offered with its scratch inside the library image instead of on the heap.
 *
 * Same arguments and semantics as mmbo_gemm_f32 without kernelId.  The caller still
 * passes A, B, C.  Limits and rules:
 *   - scratch is a fixed array of MMBO_NOALLOC_SCRATCH_BYTES bytes in the library's device
 *     image; every GPU that loads the library holds it until the process exits;
 *   - a call needs 8 * (m + n) * roundup(k, 32) bytes (each part rounded up to 1 KiB);
 *     larger problems are refused with MMBO_ERR_NOALLOC_TOO_LARGE and nothing is
 *     launched (1024 x 1024 x 1024 needs 16 MiB);
 *   - the first call on each device looks up the array's address on that device
 *     (cudaGetSymbolAddress, with that device current); make that first call before any
 *     stream capture begins;
 *   - the call performs no cudaMalloc / cudaFree and calls no allocating library routine;
 *   - all calls on a device share the one array.  Nothing in it has to start at zero:
 *     every element the GEMM reads is rewritten by the split pass of the same call, so
 *     the previous call's contents are harmless.  Two calls that overlap on the GPU
 *     (different streams) race on it: serialise them. */
#define MMBO_NOALLOC_SCRATCH_BYTES (32u << 20)
int mmbo_gemm_f32_noalloc(int transA, int transB, size_t m, size_t n, size_t k, const float* alpha,
                          const float* A, size_t lda, const float* B, size_t ldb, const float* beta,
                          float* C, size_t ldc, void* stream);

/* Self-test of the time-out path every barrier wait in the tensor-core kernels has:
 * launches one thread that waits, for at most limit_ns (<= 1 s), on a barrier nothing
 * completes.  The wait must run out, the kernel must return, and mmbo_device_status must
 * then report fault code 7 with detail 0x5e1f.  (The reference has no failure handling
 * beyond printing a status and exit(0): src/gemm/common.h:20-24.) */
int mmbo_selftest_bounded_wait(unsigned long long limit_ns, void* stream);

/* Performance tracing of the tensor-core kernels (the device-side counterpart of the
 * reference's -DDEBUG prints, src/gemm/driver.h:38-55).  mmbo_debug_trace(1, NULL, 0) arms
 * a device buffer; the following HGEMM launches record clock stamps of CTA 0 for their
 * first 64 tiles (16 words per tile: 0 tile start, 1 C requests issued, 2 accumulator
 * ready, 3 accumulator released, 4 old C arrived, 5/6 chunk stored, 8 issuer starts waiting
 * for a free accumulator, 9 got it, 10 all UMMAs issued, 11 chunk 0 in staging, 12 fenced).  mmbo_debug_trace(0, out, words)
 * copies the buffer to host memory and disarms. */
int mmbo_debug_trace(int enable, unsigned long long* out, size_t words);

/* Reads and clears the device status word of the current device (synchronises the
 * device).  *status = 0 when no kernel has recorded a fault since the last call;
 * otherwise (code << 24) | detail of the first one.  Returns MMBO_OK, a CUDA error, or
 * MMBO_ERR_DEVICE_FAULT when *status != 0. */
int mmbo_device_status(unsigned int* status);

#ifdef __cplusplus
}
#endif
#endif /* MMBO_GEMM_H_ */
