// test_gemm -- correctness harness of libmmbo_gemm.so, the counterpart of the
// reference's src/gemm/test.cc: run one kernel of the table and compare its C with the
// vendor library's on the same operands (the reference compares a hand kernel with
// rocblas_dgemm element by element at |diff| <= 1e-5, test.cc:95-120).
//
//     test_gemm [M N K] [--dtype f16|f32] [--trans NT] [--alpha a] [--beta b] [--kernel id]
//
// Here the comparison is made against two independent results: cuBLAS (cublasGemmEx,
// fp32 accumulation) and the library's one-thread-per-element kernel (id 0), with the
// relative Frobenius error and the tolerances of the benchmark specification (1e-5
// fp32, 2e-3 fp16).  The exit code is 0 only when both comparisons pass (the
// reference always exits 0).  Default shape and scalars are the reference's
// (44160 x 2048 x 384, alpha = -1, beta = 1: test.cc:20-21).
#include <cublas_v2.h>

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "mmbo_gemm.hpp"
#include "mmbo_rng.h"

namespace {

double rel_frobenius(const std::vector<float>& got, const std::vector<float>& ref) {
  double num = 0, den = 0;
  for (size_t i = 0; i < got.size(); ++i) {
    const double d = (double)got[i] - (double)ref[i];
    num += d * d;
    den += (double)ref[i] * (double)ref[i];
  }
  return den > 0 ? std::sqrt(num / den) : (num > 0 ? INFINITY : 0.0);
}

// Device C (m x n, ld = m, storage type) -> host floats.
int fetch(int dtype, const void* dC, size_t count, std::vector<float>* out) {
  out->resize(count);
  if (dtype == MMBO_DTYPE_F32) return (int)cudaMemcpy(out->data(), dC, count * 4, cudaMemcpyDeviceToHost);
  std::vector<uint16_t> tmp(count);
  const int rc = (int)cudaMemcpy(tmp.data(), dC, count * 2, cudaMemcpyDeviceToHost);
  for (size_t i = 0; i < count; ++i) (*out)[i] = mmbo_f16_bits_to_f32(tmp[i]);
  return rc;
}

}  // namespace

int main(int argc, char** argv) {
  size_t M = 44160, N = 2048, K = 384;
  int dtype = MMBO_DTYPE_F16, transA = 0, transB = 1, kernel = MMBO_KERNEL_AUTO;
  float alpha = -1.f, beta = 1.f;
  int i = 1;
  if (argc >= 4 && argv[1][0] != '-') {
    M = strtoull(argv[1], nullptr, 10);
    N = strtoull(argv[2], nullptr, 10);
    K = strtoull(argv[3], nullptr, 10);
    i = 4;
  }
  for (; i + 1 < argc; i += 2) {
    const std::string key = argv[i];
    const char* v = argv[i + 1];
    if (key == "--dtype") dtype = strcmp(v, "f32") == 0 ? MMBO_DTYPE_F32 : MMBO_DTYPE_F16;
    else if (key == "--trans" && strlen(v) == 2) { transA = v[0] == 'T'; transB = v[1] == 'T'; }
    else if (key == "--alpha") alpha = (float)atof(v);
    else if (key == "--beta") beta = (float)atof(v);
    else if (key == "--kernel") kernel = atoi(v);
    else { std::printf("unknown option %s\n", key.c_str()); return 2; }
  }
  const size_t esz = dtype == MMBO_DTYPE_F32 ? 4 : 2;
  const size_t rowsA = transA ? K : M, colsA = transA ? M : K;
  const size_t rowsB = transB ? N : K, colsB = transB ? K : N;
  const size_t lda = rowsA, ldb = rowsB, ldc = M;
  void *dA, *dB, *dC0, *dC1, *dC2, *dC3;
  MMBO_CHECK(cudaMalloc(&dA, lda * colsA * esz));
  MMBO_CHECK(cudaMalloc(&dB, ldb * colsB * esz));
  MMBO_CHECK(cudaMalloc(&dC0, ldc * N * esz));  // initial C
  MMBO_CHECK(cudaMalloc(&dC1, ldc * N * esz));  // kernel under test
  MMBO_CHECK(cudaMalloc(&dC2, ldc * N * esz));  // vendor library
  MMBO_CHECK(cudaMalloc(&dC3, ldc * N * esz));  // simplest kernel of the table
  auto fill = [&](void* p, size_t rows, size_t cols, unsigned mat) {
    return dtype == MMBO_DTYPE_F32
               ? mmbo_fill_f32((float*)p, rows, cols, rows, 1234, mat, MMBO_DIST_UNIFORM_PM1, 1.f, 0, 0, rows, nullptr)
               : mmbo_fill_f16(p, rows, cols, rows, 1234, mat, MMBO_DIST_UNIFORM_PM1, 1.f, 0, 0, rows, nullptr);
  };
  MMBO_CHECK(fill(dA, rowsA, colsA, MMBO_MAT_A));
  MMBO_CHECK(fill(dB, rowsB, colsB, MMBO_MAT_B));
  MMBO_CHECK(fill(dC0, M, N, MMBO_MAT_C));
  for (void* c : {dC1, dC2, dC3}) MMBO_CHECK(cudaMemcpy(c, dC0, ldc * N * esz, cudaMemcpyDeviceToDevice));

  int id = kernel;
  if (id == MMBO_KERNEL_AUTO) id = mmbo_select_kernel(dtype, transA, transB, M, N, K, dA, lda, dB, ldb, dC1, ldc);
  MMBO_CHECK(id < 0 ? id : 0);
  std::printf("kernel under test: %d %s\n", id, mmbo_kernel_name(dtype, id));

  cudaEvent_t ev0, ev1;
  float seconds;
  MMBO_GPU_TIMER_START(seconds, ev0, ev1, nullptr);
  MMBO_CHECK(mmbo::launchGemm(dtype, transA, transB, M, N, K, &alpha, dA, lda, dB, ldb, &beta, dC1, ldc, id));
  MMBO_GPU_TIMER_END(seconds, ev0, ev1, nullptr);
  std::printf("time = %f s, %.4f TFLOP/s (first launch, includes one-time set-up)\n", seconds,
              1e-12 * 2.0 * M * N * K / seconds);
  MMBO_CHECK(mmbo::launchGemm(dtype, transA, transB, M, N, K, &alpha, dA, lda, dB, ldb, &beta, dC3, ldc, 0));

  cublasHandle_t h;
  if (cublasCreate(&h) != CUBLAS_STATUS_SUCCESS) { std::fprintf(stderr, "cublasCreate failed\n"); return 1; }
  const cudaDataType_t dt = dtype == MMBO_DTYPE_F32 ? CUDA_R_32F : CUDA_R_16F;
  if (cublasGemmEx(h, transA ? CUBLAS_OP_T : CUBLAS_OP_N, transB ? CUBLAS_OP_T : CUBLAS_OP_N, (int)M, (int)N, (int)K,
                   &alpha, dA, dt, (int)lda, dB, dt, (int)ldb, &beta, dC2, dt, (int)ldc,
                   dtype == MMBO_DTYPE_F32 ? CUBLAS_COMPUTE_32F_PEDANTIC : CUBLAS_COMPUTE_32F,
                   CUBLAS_GEMM_DEFAULT) != CUBLAS_STATUS_SUCCESS) {
    std::fprintf(stderr, "cublasGemmEx failed\n");
    return 1;
  }
  MMBO_CHECK(cudaDeviceSynchronize());
  unsigned int fault = 0;
  MMBO_CHECK(mmbo_device_status(&fault));

  std::vector<float> c1, c2, c3;
  MMBO_CHECK(fetch(dtype, dC1, ldc * N, &c1));
  MMBO_CHECK(fetch(dtype, dC2, ldc * N, &c2));
  MMBO_CHECK(fetch(dtype, dC3, ldc * N, &c3));
  std::printf("C(0,0) C(1,0) C(m-1,n-1): test %.5f %.5f %.5f | cublas %.5f %.5f %.5f\n", c1[0], c1[1],
              c1[ldc * N - 1], c2[0], c2[1], c2[ldc * N - 1]);
  const double tol = dtype == MMBO_DTYPE_F32 ? 1e-5 : 2e-3;
  const double e_vendor = rel_frobenius(c1, c2), e_simple = rel_frobenius(c1, c3);
  std::printf("relative Frobenius error vs cuBLAS = %.3e, vs kernel 0 = %.3e (tolerance %.1e)\n", e_vendor,
              e_simple, tol);
  const bool ok = e_vendor <= tol && e_simple <= tol;
  std::printf(ok ? "results match\n" : "results DIFFER\n");
  cublasDestroy(h);
  for (void* p : {dA, dB, dC0, dC1, dC2, dC3}) cudaFree(p);
  return ok ? 0 : 1;
}
