// benchmark -- command-line harness of libmmbo_gemm.so, the counterpart of the
// reference's src/gemm/benchmark.cc.  The positional form is the reference's
// (src/gemm/benchmark.cc:27-35):
//
//     benchmark <type> M N K lda ldb ldc [options]
//
//   type 0  the library's own choice of kernel (the reference's "naive" hand-tuned arm,
//           benchmark.cc:72-88)
//   type 1  every kernel of the table in turn, best one reported (the reference's sweep
//           over its Tensile table, benchmark.cc:89-109)
//   type 2  the vendor library (cuBLAS here, rocBLAS in the reference, benchmark.cc:110-117)
//
//   options: --dtype f16|f32|f64 (default f16; f64 is the reference's own type)   --trans NN|NT|TN|TT (default NT)
//            --alpha a --beta b (defaults -1, 1: the reference's HPL update, benchmark.cc:21)
//            --kernel id (type 0 only)  --seed s  --iters n (timed launches, default 20)
//
// Differences from the reference that are deliberate: operands are generated on the
// device from a seed (the reference fills them with unseeded rand()); warm-up and a loop
// of timed launches instead of one; nothing but the kernel inside the timed region (the
// reference times hipModuleLoad as well, driver.h:41); errors are reported and returned.
// One line per result, in the reference's field order:
//   <arm>(<trans>): kernel, m, n, k, lda, ldb, time, tflops, efficiency
#include <cublas_v2.h>

#include <cstdlib>
#include <cstring>
#include <string>

#include "mmbo_gemm.hpp"
#include "mmbo_rng.h"

namespace {

struct Options {
  int type = -1;
  size_t M = 44160, N = 2048, K = 384, lda = 0, ldb = 0, ldc = 0;
  int dtype = MMBO_DTYPE_F16;
  int transA = 0, transB = 1;
  float alpha = -1.f, beta = 1.f;
  int kernel = MMBO_KERNEL_AUTO;
  unsigned long long seed = 1234;
  int iters = 20;
};

bool parse(int argc, char** argv, Options* o) {
  if (argc < 8) return false;
  o->type = atoi(argv[1]);
  o->M = strtoull(argv[2], nullptr, 10);
  o->N = strtoull(argv[3], nullptr, 10);
  o->K = strtoull(argv[4], nullptr, 10);
  o->lda = strtoull(argv[5], nullptr, 10);
  o->ldb = strtoull(argv[6], nullptr, 10);
  o->ldc = strtoull(argv[7], nullptr, 10);
  for (int i = 8; i + 1 < argc; i += 2) {
    const std::string key = argv[i];
    const char* v = argv[i + 1];
    if (key == "--dtype") o->dtype = strcmp(v, "f32") == 0 ? MMBO_DTYPE_F32 : strcmp(v, "f64") == 0 ? MMBO_DTYPE_F64 : MMBO_DTYPE_F16;
    else if (key == "--trans" && strlen(v) == 2) { o->transA = v[0] == 'T'; o->transB = v[1] == 'T'; }
    else if (key == "--alpha") o->alpha = (float)atof(v);
    else if (key == "--beta") o->beta = (float)atof(v);
    else if (key == "--kernel") o->kernel = atoi(v);
    else if (key == "--seed") o->seed = strtoull(v, nullptr, 10);
    else if (key == "--iters") o->iters = atoi(v);
    else return false;
  }
  return o->type >= 0 && o->type <= 2 && o->iters > 0;
}

// Peak the "efficiency" column divides by (the reference divides by a constant 6.5
// TFLOP/s, benchmark.cc:86): dense fp16 tensor peak, or SMs x 128 lanes x 2 x clock.
double peak_tflops(int dtype) {
  if (dtype == MMBO_DTYPE_F16) return 2250.0;
  int dev = 0, sms = 148, khz = 1965000;
  const double lanes = dtype == MMBO_DTYPE_F64 ? 64.0 : 128.0;  // FMA lanes per SM per clock
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev);
  return sms * lanes * 2.0 * khz * 1e3 / 1e12;
}

}  // namespace

int main(int argc, char** argv) {
  Options o;
  if (!parse(argc, argv, &o)) {
    std::printf("usage: benchmark <type 0|1|2> M N K lda ldb ldc [--dtype f16|f32] [--trans NT] "
                "[--alpha a] [--beta b] [--kernel id] [--seed s] [--iters n]\n");
    return 2;
  }
  const size_t esz = o.dtype == MMBO_DTYPE_F32 ? 4 : o.dtype == MMBO_DTYPE_F64 ? 8 : 2;
  const size_t rowsA = o.transA ? o.K : o.M, colsA = o.transA ? o.M : o.K;
  const size_t rowsB = o.transB ? o.N : o.K, colsB = o.transB ? o.K : o.N;
  void *dA = nullptr, *dB = nullptr, *dC = nullptr;
  MMBO_CHECK(cudaMalloc(&dA, o.lda * colsA * esz));
  MMBO_CHECK(cudaMalloc(&dB, o.ldb * colsB * esz));
  MMBO_CHECK(cudaMalloc(&dC, o.ldc * o.N * esz));
  auto fill = [&](void* p, size_t rows, size_t cols, size_t ld, unsigned mat) {
    if (ld < rows) return (int)MMBO_ERR_BAD_LDC;
    cudaMemset(p, 0, ld * cols * esz);
    if (o.dtype == MMBO_DTYPE_F64)
      return mmbo_fill_f64((double*)p, rows, cols, ld, o.seed, mat, MMBO_DIST_UNIFORM_PM1, 1.f, 0, 0, rows, nullptr);
    return o.dtype == MMBO_DTYPE_F32
               ? mmbo_fill_f32((float*)p, rows, cols, ld, o.seed, mat, MMBO_DIST_UNIFORM_PM1, 1.f, 0, 0, rows, nullptr)
               : mmbo_fill_f16(p, rows, cols, ld, o.seed, mat, MMBO_DIST_UNIFORM_PM1, 1.f, 0, 0, rows, nullptr);
  };
  MMBO_CHECK(fill(dA, rowsA, colsA, o.lda, MMBO_MAT_A));
  MMBO_CHECK(fill(dB, rowsB, colsB, o.ldb, MMBO_MAT_B));
  MMBO_CHECK(fill(dC, o.M, o.N, o.ldc, MMBO_MAT_C));

  const char trans[3] = {o.transA ? 'T' : 'N', o.transB ? 'T' : 'N', 0};
  const char* prefix = o.dtype == MMBO_DTYPE_F32 ? "s" : o.dtype == MMBO_DTYPE_F64 ? "d" : "h";
  double alpha64 = o.alpha, beta64 = o.beta;
  // one call of the library for the chosen dtype (binary64 takes double scalars, like the reference)
  auto gemm_call = [&](int id) -> int {
    if (o.dtype == MMBO_DTYPE_F64)
      return mmbo::launchGemm(o.dtype, o.transA, o.transB, o.M, o.N, o.K, &alpha64, dA, o.lda, dB, o.ldb, &beta64, dC,
                              o.ldc, id);
    return mmbo::launchGemm(o.dtype, o.transA, o.transB, o.M, o.N, o.K, &o.alpha, dA, o.lda, dB, o.ldb, &o.beta, dC,
                            o.ldc, id);
  };
  const double flops = 2.0 * (double)o.M * (double)o.N * (double)o.K;
  const double peak = peak_tflops(o.dtype);
  cudaEvent_t ev0, ev1;
  float seconds = 0.f;

  auto time_kernel = [&](int id, double* tflops) -> int {
    for (int w = 0; w < 3; ++w) {
      int rc = gemm_call(id);
      if (rc) return rc;
    }
    MMBO_GPU_TIMER_START(seconds, ev0, ev1, nullptr);
    for (int it = 0; it < o.iters; ++it) gemm_call(id);
    MMBO_GPU_TIMER_END(seconds, ev0, ev1, nullptr);
    seconds /= o.iters;
    *tflops = 1e-12 * flops / seconds;
    return 0;
  };

  if (o.type == 0) {
    int id = o.kernel;
    double tflops = 0;
    MMBO_CHECK(time_kernel(id, &tflops));
    if (id == MMBO_KERNEL_AUTO) id = mmbo_last_kernel(o.dtype);  // the row the library chose for these arguments, beta included
    MMBO_CHECK(id < 0 ? id : 0);
    std::printf("%s\n", mmbo_kernel_name(o.dtype, id));
    std::printf("mmbo_%sgemm(%s): kernel, m, n, k, lda, ldb, time, tflops, efficiency = %d, %zu, %zu, %zu, %zu, "
                "%zu, %.6f, %.5f, %.2f%%\n", prefix, trans, id, o.M, o.N, o.K, o.lda, o.ldb, seconds, tflops,
                tflops / peak * 100);
  } else if (o.type == 1) {
    double best = 0;
    float best_s = 0;
    int best_id = -1;
    for (const auto& k : mmbo::kernel_table(o.dtype)) {
      double tflops = 0;
      const int rc = time_kernel(k.id, &tflops);
      if (rc == MMBO_ERR_KERNEL_UNSUITABLE) continue;  // operands this row cannot address
      MMBO_CHECK(rc);
      std::printf("  id %d %-52s %.6f s %.4f TFLOP/s\n", k.id, k.name.c_str(), seconds, tflops);
      if (tflops > best) { best = tflops; best_id = k.id; best_s = seconds; }
    }
    std::printf("table_%sgemm(%s): kernel, m, n, k, lda, ldb, time, tflops, efficiency = %d, %zu, %zu, %zu, %zu, "
                "%zu, %.6f, %.5f, %.2f%%\n", prefix, trans, best_id, o.M, o.N, o.K, o.lda, o.ldb, best_s, best,
                best / peak * 100);
  } else {
    cublasHandle_t h;
    if (cublasCreate(&h) != CUBLAS_STATUS_SUCCESS) { std::fprintf(stderr, "cublasCreate failed\n"); return 1; }
    const cudaDataType_t dt = o.dtype == MMBO_DTYPE_F32 ? CUDA_R_32F : o.dtype == MMBO_DTYPE_F64 ? CUDA_R_64F : CUDA_R_16F;
    auto call = [&]() {
      if (o.dtype == MMBO_DTYPE_F64)
        return cublasDgemm(h, o.transA ? CUBLAS_OP_T : CUBLAS_OP_N, o.transB ? CUBLAS_OP_T : CUBLAS_OP_N, (int)o.M,
                           (int)o.N, (int)o.K, &alpha64, (const double*)dA, (int)o.lda, (const double*)dB, (int)o.ldb,
                           &beta64, (double*)dC, (int)o.ldc);
      return cublasGemmEx(h, o.transA ? CUBLAS_OP_T : CUBLAS_OP_N, o.transB ? CUBLAS_OP_T : CUBLAS_OP_N, (int)o.M,
                          (int)o.N, (int)o.K, &o.alpha, dA, dt, (int)o.lda, dB, dt, (int)o.ldb, &o.beta, dC, dt,
                          (int)o.ldc, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
    };
    for (int w = 0; w < 3; ++w)
      if (call() != CUBLAS_STATUS_SUCCESS) { std::fprintf(stderr, "cublasGemmEx failed\n"); return 1; }
    MMBO_GPU_TIMER_START(seconds, ev0, ev1, nullptr);
    for (int it = 0; it < o.iters; ++it) call();
    MMBO_GPU_TIMER_END(seconds, ev0, ev1, nullptr);
    seconds /= o.iters;
    const double tflops = 1e-12 * flops / seconds;
    std::printf("cublas_%sgemm(%s): m, n, k, lda, ldb, time, tflops, efficiency = %zu, %zu, %zu, %zu, %zu, %.6f, "
                "%.5f, %.2f%%\n", prefix, trans, o.M, o.N, o.K, o.lda, o.ldb, seconds, tflops, tflops / peak * 100);
    cublasDestroy(h);
  }
  unsigned int fault = 0;
  MMBO_CHECK(mmbo_device_status(&fault));
  cudaFree(dA);
  cudaFree(dB);
  cudaFree(dC);
  return 0;
}
