// mmbo_gemm.hpp -- C++ face of libmmbo_gemm.so for host programs written against the
// reference's headers.  Header-only, inline (the reference's gemm.h defines non-inline
// functions in a header and can only be included from one translation unit).
//
//   reference                               here
//   ---------------------------------------------------------------------------------
//   dgemm_NT(m,n,k,alpha,A,lda,B,ldb,       sgemm_NT / sgemm_NN / sgemm_TN / sgemm_TT,
//            beta,C,ldc,kernelId)            hgemm_NT / hgemm_NN / hgemm_TN / hgemm_TT:
//     src/gemm/gemm.h:47-48                  same argument order, kernelId last
//   naive_dgemm(...)  src/gemm/gemm.h:4-5    same wrappers with kernelId = MMBO_KERNEL_AUTO
//   launchGemm(...)   src/gemm/driver.h:15   mmbo::launchGemm(dtype, transA, transB, ...)
//   kernels[] / kernel_parameters[][3]       mmbo::kernel_table(dtype)
//     src/gemm/constants.h:4-135
//   GPU_TIMER_START / GPU_TIMER_END          MMBO_GPU_TIMER_START / MMBO_GPU_TIMER_END
//     src/gemm/common.h:4-18                 (seconds, CUDA events on a stream)
//   HIP_CHECK (prints, exit(0))              MMBO_CHECK (prints, returns the status)
//     src/gemm/common.h:20-24
//
// alpha and beta are host pointers, A/B/C device pointers, exactly as in the reference.
// For fp16 the scalars are float (the accumulator type).
#ifndef MMBO_GEMM_HPP_
#define MMBO_GEMM_HPP_

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <string>
#include <vector>

#include "mmbo_gemm.h"

namespace mmbo {

struct KernelInfo {
  int id;
  std::string name;
  int MT0, MT1, threads, DepthU, stages, ctaGroup, wgm;
  bool tensorCores;
};

// The kernel table of one dtype, in kernelId order.
inline std::vector<KernelInfo> kernel_table(int dtype) {
  std::vector<KernelInfo> out;
  const int n = mmbo_num_kernels(dtype);
  for (int i = 0; i < n; ++i) {
    int p[8];
    if (mmbo_kernel_params(dtype, i, p) != MMBO_OK) continue;
    out.push_back(KernelInfo{i, mmbo_kernel_name(dtype, i), p[0], p[1], p[2], p[3], p[4], p[5], p[6], p[7] != 0});
  }
  return out;
}

// Low-level entry: validates, selects (kernelId = MMBO_KERNEL_AUTO) or forces a table row
// and queues the kernel on `stream`.  Returns the library status; nothing is loaded from
// disk and nothing is printed.
inline int launchGemm(int dtype, int transA, int transB, size_t m, size_t n, size_t k, const float* alpha,
                      const void* A, size_t lda, const void* B, size_t ldb, const float* beta, void* C,
                      size_t ldc, int kernelId = MMBO_KERNEL_AUTO, cudaStream_t stream = nullptr) {
  if (dtype == MMBO_DTYPE_F32)
    return mmbo_gemm_f32(transA, transB, m, n, k, alpha, static_cast<const float*>(A), lda,
                         static_cast<const float*>(B), ldb, beta, static_cast<float*>(C), ldc, kernelId, stream);
  if (dtype == MMBO_DTYPE_F16)
    return mmbo_gemm_f16(transA, transB, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, kernelId, stream);
  return MMBO_ERR_BAD_DTYPE;  // binary64 takes double scalars: the overload below
}

// The same entry for binary64, the reference's own data type (its launchGemm is what
// dgemm_NT calls: src/gemm/gemm.h:95): the scalars are double, as in the reference.
inline int launchGemm(int dtype, int transA, int transB, size_t m, size_t n, size_t k, const double* alpha,
                      const void* A, size_t lda, const void* B, size_t ldb, const double* beta, void* C,
                      size_t ldc, int kernelId = MMBO_KERNEL_AUTO, cudaStream_t stream = nullptr) {
  if (dtype != MMBO_DTYPE_F64) return MMBO_ERR_BAD_DTYPE;  // fp32 / fp16 take float scalars
  return mmbo_gemm_f64(transA, transB, m, n, k, alpha, static_cast<const double*>(A), lda,
                       static_cast<const double*>(B), ldb, beta, static_cast<double*>(C), ldc, kernelId, stream);
}

}  // namespace mmbo

#define MMBO_DEFINE_GEMM(NAME, TA, TB)                                                                       \
  inline int s##NAME(size_t m, size_t n, size_t k, float* alpha, const float* A, size_t lda, const float* B, \
                     size_t ldb, float* beta, float* C, size_t ldc, int kernelId = MMBO_KERNEL_AUTO,         \
                     cudaStream_t stream = nullptr) {                                                        \
    return mmbo_gemm_f32(TA, TB, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, kernelId, stream);            \
  }                                                                                                          \
  inline int h##NAME(size_t m, size_t n, size_t k, float* alpha, const __half* A, size_t lda,                \
                     const __half* B, size_t ldb, float* beta, __half* C, size_t ldc,                        \
                     int kernelId = MMBO_KERNEL_AUTO, cudaStream_t stream = nullptr) {                       \
    return mmbo_gemm_f16(TA, TB, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, kernelId, stream);            \
  }
MMBO_DEFINE_GEMM(gemm_NN, 0, 0)
MMBO_DEFINE_GEMM(gemm_NT, 0, 1)
MMBO_DEFINE_GEMM(gemm_TN, 1, 0)
MMBO_DEFINE_GEMM(gemm_TT, 1, 1)
#undef MMBO_DEFINE_GEMM

// The reference's own entry points, name for name and argument for argument
// (src/gemm/gemm.h:47-48 and :4-5): binary64, NT layout, void return.  A failure is
// reported on stderr; the process keeps running.
inline void dgemm_NT(size_t m, size_t n, size_t k, double* alpha, const double* A, size_t lda, const double* B,
                     size_t ldb, double* beta, double* C, size_t ldc, int kernelId) {
  const int rc = mmbo_gemm_f64(0, 1, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, kernelId, nullptr);
  if (rc != 0) std::fprintf(stderr, "dgemm_NT: status %d: %s\n", rc, mmbo_status_string(rc));
}
inline void naive_dgemm(size_t m, size_t n, size_t k, double* alpha, const double* A, size_t lda, const double* B,
                        size_t ldb, double* beta, double* C, size_t ldc, int kernelId) {
  dgemm_NT(m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, kernelId);
}
inline int dgemm(int transA, int transB, size_t m, size_t n, size_t k, double* alpha, const double* A, size_t lda,
                 const double* B, size_t ldb, double* beta, double* C, size_t ldc,
                 int kernelId = MMBO_KERNEL_AUTO, cudaStream_t stream = nullptr) {
  return mmbo_gemm_f64(transA, transB, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, kernelId, stream);
}

// Event-pair timer on a stream; elapsed time in seconds, like the reference's macros.
#define MMBO_GPU_TIMER_START(elapsed, ev_start, ev_stop, stream) \
  do {                                                           \
    (elapsed) = 0.0f;                                            \
    cudaEventCreate(&(ev_start));                                \
    cudaEventCreate(&(ev_stop));                                 \
    cudaEventRecord((ev_start), (stream));                       \
  } while (0)

#define MMBO_GPU_TIMER_END(elapsed, ev_start, ev_stop, stream)   \
  do {                                                           \
    cudaEventRecord((ev_stop), (stream));                        \
    cudaEventSynchronize((ev_stop));                             \
    cudaEventElapsedTime(&(elapsed), (ev_start), (ev_stop));     \
    (elapsed) /= 1000.0f;                                        \
    cudaEventDestroy((ev_start));                                \
    cudaEventDestroy((ev_stop));                                 \
  } while (0)

// Reports a failed library or CUDA call and hands the status back to the caller.
#define MMBO_CHECK(expr)                                                                            \
  do {                                                                                              \
    const int mmbo_status_ = static_cast<int>(expr);                                                \
    if (mmbo_status_ != 0) {                                                                        \
      std::fprintf(stderr, "%s:%d: status %d: %s\n", __FILE__, __LINE__, mmbo_status_,              \
                   mmbo_status_string(mmbo_status_));                                               \
      return mmbo_status_ > 0 ? mmbo_status_ : -mmbo_status_;                                       \
    }                                                                                               \
  } while (0)

#endif  // MMBO_GEMM_HPP_
