// float64 product C = alpha * A @ B + beta * C behind the reference's second
// device BLAS entry (numba_mlir/mlir/math_runtime.py:36-40 registers
// "mkl_gemm_float64_device" beside the float32 one; the SYCL side is
// numba_mlir_gpu_runtime_sycl/lib/NumpyLinalg.cpp:67-176).
//
// B200 has no fast float64 tensor path, so this is a register-tiled CUDA-core
// kernel: a block of 256 threads owns a 64 x 64 tile of C, a thread a 4 x 4
// piece of it; A and B travel through shared memory 16 columns of K at a time
// (any row/column strides: both operands are read with their own strides, so
// transposed views need no copy).  Sums run over k in index order.
#include "gpu_common.h"

#include <cuda_runtime.h>

#include <cstdint>

#define GPUX_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

constexpr int kTileM = 64, kTileN = 64, kTileK = 16, kThreads = 256;

struct GemmF64 {
  const double *a, *b;
  double *c;
  int64_t M, N, K;
  int64_t a_r, a_k; // element (i, k) of A at a[i * a_r + k * a_k]
  int64_t b_k, b_c; // element (k, j) of B at b[k * b_k + j * b_c]
  int64_t c_r, c_c;
  double alpha, beta;
};

__global__ void __launch_bounds__(kThreads) nmb_gemm_f64(const GemmF64 p) {
  __shared__ double sa[kTileK][kTileM + 1];
  __shared__ double sb[kTileK][kTileN + 1];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4; // 16 x 16 threads, 4 x 4 outputs each
  const int64_t i0 = (int64_t)blockIdx.y * kTileM, j0 = (int64_t)blockIdx.x * kTileN;
  double acc[4][4] = {};
  for (int64_t k0 = 0; k0 < p.K; k0 += kTileK) {
    // 64 x 16 elements of A and 16 x 64 of B: four of each per thread
    for (int e = threadIdx.x; e < kTileM * kTileK; e += kThreads) {
      const int kk = e % kTileK, ii = e / kTileK;
      const int64_t i = i0 + ii, k = k0 + kk;
      sa[kk][ii] = (i < p.M && k < p.K) ? p.a[i * p.a_r + k * p.a_k] : 0.0;
    }
    for (int e = threadIdx.x; e < kTileN * kTileK; e += kThreads) {
      const int jj = e % kTileN, kk = e / kTileN;
      const int64_t j = j0 + jj, k = k0 + kk;
      sb[kk][jj] = (j < p.N && k < p.K) ? p.b[k * p.b_k + j * p.b_c] : 0.0;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kTileK; ++kk) {
      double av[4], bv[4];
#pragma unroll
      for (int r = 0; r < 4; ++r)
        av[r] = sa[kk][ty * 4 + r];
#pragma unroll
      for (int c = 0; c < 4; ++c)
        bv[c] = sb[kk][tx + 16 * c];
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c)
          acc[r][c] = fma(av[r], bv[c], acc[r][c]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int64_t i = i0 + ty * 4 + r;
    if (i >= p.M)
      continue;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int64_t j = j0 + tx + 16 * c;
      if (j >= p.N)
        continue;
      double *dst = p.c + i * p.c_r + j * p.c_c;
      const double v = p.alpha * acc[r][c];
      *dst = p.beta == 0.0 ? v : fma(p.beta, *dst, v);
    }
  }
}

bool enqueue(void *queue, const GPUXMemref2d *a, const GPUXMemref2d *b, double alpha, double beta,
             GPUXMemref2d *c) {
  if (!queue || !a || !b || !c) {
    nmb::setError("mkl_gemm_float64_device: null argument");
    return false;
  }
  if (a->dims[1] != b->dims[0] || c->dims[0] != a->dims[0] || c->dims[1] != b->dims[1]) {
    nmb::setError("mkl_gemm_float64_device: shape mismatch a (%zu,%zu), b (%zu,%zu), c (%zu,%zu)",
                  a->dims[0], a->dims[1], b->dims[0], b->dims[1], c->dims[0], c->dims[1]);
    return false;
  }
  nmb::QueueView qv;
  if (!nmb::queueView(queue, &qv))
    return false;
  GemmF64 p;
  p.a = a->data + a->offset;
  p.b = b->data + b->offset;
  p.c = c->data + c->offset;
  p.M = (int64_t)a->dims[0];
  p.K = (int64_t)a->dims[1];
  p.N = (int64_t)b->dims[1];
  p.a_r = (int64_t)a->strides[0];
  p.a_k = (int64_t)a->strides[1];
  p.b_k = (int64_t)b->strides[0];
  p.b_c = (int64_t)b->strides[1];
  p.c_r = (int64_t)c->strides[0];
  p.c_c = (int64_t)c->strides[1];
  p.alpha = alpha;
  p.beta = beta;
  if (p.M == 0 || p.N == 0)
    return true;
  const int64_t gy = (p.M + kTileM - 1) / kTileM, gx = (p.N + kTileN - 1) / kTileN;
  if (gy > 65535) {
    nmb::setError("mkl_gemm_float64_device: more than 65535 row tiles");
    return false;
  }
  cudaSetDevice(qv.device);
  nmb_gemm_f64<<<dim3((unsigned)gx, (unsigned)gy), kThreads, 0, static_cast<cudaStream_t>(qv.stream)>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    nmb::setError("mkl_gemm_float64_device: launch failed: %s", cudaGetErrorString(e));
    return false;
  }
  nmb::noteLaunch();
  return true;
}

} // namespace

// Blocking, like the reference's call (NumpyLinalg.cpp:143-146 waits on the oneMKL event).
GPUX_EXPORT void _mlir_ciface_mkl_gemm_float64_device(void *queue, const GPUXMemref2d *a, const GPUXMemref2d *b,
                                                      double alpha, double beta, GPUXMemref2d *c) {
  if (!enqueue(queue, a, b, alpha, beta, c))
    return;
  nmb::QueueView qv;
  if (nmb::queueView(queue, &qv)) {
    cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(qv.stream));
    if (e != cudaSuccess)
      nmb::setError("mkl_gemm_float64_device failed: %s", cudaGetErrorString(e));
  }
}

GPUX_EXPORT void mkl_gemm_float64_device(void *q, const GPUXMemref2d *a, const GPUXMemref2d *b, double alpha,
                                         double beta, GPUXMemref2d *c) {
  _mlir_ciface_mkl_gemm_float64_device(q, a, b, alpha, beta, c);
}

// The same product without the host-side wait; returns an event.
GPUX_EXPORT void *_mlir_ciface_nmb_gemm_float64_device_async(void *queue, const GPUXMemref2d *a,
                                                             const GPUXMemref2d *b, double alpha, double beta,
                                                             GPUXMemref2d *c) {
  if (!enqueue(queue, a, b, alpha, beta, c))
    return nullptr;
  return nmb::recordEventOn(queue);
}
