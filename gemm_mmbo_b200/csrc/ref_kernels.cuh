// Simple kernels: the obviously-correct GEMM (kernel id 0 of every dtype; also the
// path taken for operands the fast kernels cannot address), the k == 0 scaling kernel
// and the seeded operand generators.
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

#include "../../include/mmbo_rng.h"

namespace mmbo {

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ double from_f32<double>(float v) { return (double)v; }

// One thread per C element, 32 x 8 thread blocks (32 consecutive rows per warp so that
// C and non-transposed A accesses coalesce).  fp32 accumulation in increasing l.
// The write rule is the reference's TYPE_MAC_WRITE (src/gemm/ref/Kernels.cpp:87):
// beta == 0 stores alpha*acc without reading C.
template <typename T>
__global__ void gemm_simple_kernel(int transA, int transB, size_t m, size_t n, size_t k, float alpha,
                                   const T* __restrict__ A, size_t lda, const T* __restrict__ B,
                                   size_t ldb, float beta, T* __restrict__ C, size_t ldc, size_t batch_a,
                                   size_t batch_b, size_t batch_c) {
  A += (size_t)blockIdx.z * batch_a;  // problem blockIdx.z of a strided batch
  B += (size_t)blockIdx.z * batch_b;
  C += (size_t)blockIdx.z * batch_c;
  const size_t i = (size_t)blockIdx.x * 32 + threadIdx.x;
  const size_t j = (size_t)blockIdx.y * 8 + threadIdx.y;
  if (i >= m || j >= n) return;
  float acc = 0.0f;
  for (size_t l = 0; l < k; ++l) {
    const float a = to_f32<T>(transA ? A[l + i * lda] : A[i + l * lda]);
    const float b = to_f32<T>(transB ? B[j + l * ldb] : B[l + j * ldb]);
    acc = fmaf(a, b, acc);
  }
  float r = alpha * acc;
  if (beta != 0.0f) r = fmaf(beta, to_f32<T>(C[i + j * ldc]), r);
  C[i + j * ldc] = from_f32<T>(r);
}

// binary64 variant of the kernel above (accumulation and scalars in binary64).
__global__ void gemm_simple_f64_kernel(int transA, int transB, size_t m, size_t n, size_t k, double alpha,
                                       const double* __restrict__ A, size_t lda, const double* __restrict__ B,
                                       size_t ldb, double beta, double* __restrict__ C, size_t ldc, size_t batch_a,
                                       size_t batch_b, size_t batch_c) {
  A += (size_t)blockIdx.z * batch_a;
  B += (size_t)blockIdx.z * batch_b;
  C += (size_t)blockIdx.z * batch_c;
  const size_t i = (size_t)blockIdx.x * 32 + threadIdx.x;
  const size_t j = (size_t)blockIdx.y * 8 + threadIdx.y;
  if (i >= m || j >= n) return;
  double acc = 0.0;
  for (size_t l = 0; l < k; ++l) {
    const double a = transA ? A[l + i * lda] : A[i + l * lda];
    const double b = transB ? B[j + l * ldb] : B[l + j * ldb];
    acc = fma(a, b, acc);
  }
  double r = alpha * acc;
  if (beta != 0.0) r = fma(beta, C[i + j * ldc], r);
  C[i + j * ldc] = r;
}

__global__ void scale_c_f64_kernel(size_t m, size_t n, double beta, double* __restrict__ C, size_t ldc,
                                   size_t batch_c) {
  C += (size_t)blockIdx.z * batch_c;
  const size_t i = (size_t)blockIdx.x * 32 + threadIdx.x;
  const size_t j = (size_t)blockIdx.y * 8 + threadIdx.y;
  if (i >= m || j >= n) return;
  C[i + j * ldc] = beta != 0.0 ? beta * C[i + j * ldc] : 0.0;
}

// k == 0: C = beta*C (or zero when beta == 0).
template <typename T>
__global__ void scale_c_kernel(size_t m, size_t n, float beta, T* __restrict__ C, size_t ldc, size_t batch_c) {
  C += (size_t)blockIdx.z * batch_c;
  const size_t i = (size_t)blockIdx.x * 32 + threadIdx.x;
  const size_t j = (size_t)blockIdx.y * 8 + threadIdx.y;
  if (i >= m || j >= n) return;
  float r = 0.0f;
  if (beta != 0.0f) r = beta * to_f32<T>(C[i + j * ldc]);
  C[i + j * ldc] = from_f32<T>(r);
}

// Seeded generator: element (i, j) of the rows x cols window of a column-major array
// gets the value of logical element (row0 + i, col0 + j) of a matrix with total_rows
// rows.  Padding rows (i >= rows) are not written.
template <typename T>
__global__ void fill_kernel(T* __restrict__ dst, size_t rows, size_t cols, size_t ld, uint64_t seed,
                            uint32_t mat, int dist, float scale, size_t row0, size_t col0,
                            size_t total_rows) {
  const size_t total = rows * cols;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t i = idx % rows, j = idx / rows;
    const float v = mmbo_rng_value(seed, mat, row0 + i, col0 + j, total_rows, dist, scale);
    dst[i + j * ld] = from_f32<T>(v);
  }
}

}  // namespace mmbo
