// float64 product C = alpha * A @ B + beta * C behind the reference's second
// device BLAS entry (numba_mlir/mlir/math_runtime.py:36-40 registers
// "mkl_gemm_float64_device" beside the float32 one; the SYCL side is
// numba_mlir_gpu_runtime_sycl/lib/NumpyLinalg.cpp:67-176).
//
// B200 has no fast float64 tensor path, so this is a register-tiled CUDA-core
// kernel: a block of 256 threads owns a 128 x 128 tile of C, a thread an 8 x 8
// piece of it; A and B travel through shared memory 8 columns of K at a time
// (any row/column strides: both operands are read with their own strides, so
// transposed views need no copy).  Sums run over k in index order.
#include "gpu_common.h"

#include <cuda_runtime.h>

#include <cstdint>

#define GPUX_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

constexpr int kTileM = 128, kTileN = 128, kTileK = 8, kThreads = 256;

struct GemmF64 {
  const double *a, *b;
  double *c;
  int64_t M, N, K;
  int64_t a_r, a_k; // element (i, k) of A at a[i * a_r + k * a_k]
  int64_t b_k, b_c; // element (k, j) of B at b[k * b_k + j * b_c]
  int64_t c_r, c_c;
  double alpha, beta;
};

// A thread owns the 8 x 8 outputs at rows ty*4 + {0..3} and 64 + ty*4 + {0..3},
// columns tx*4 + {0..3} and 64 + tx*4 + {0..3}: per k step it reads four pairs
// of doubles (16-byte shared loads) for 64 fused multiply-adds.  The next K
// slice is fetched into registers while the current one is multiplied.
__global__ void __launch_bounds__(kThreads) nmb_gemm_f64(const GemmF64 p) {
  __shared__ __align__(16) double sa[kTileK][kTileM];
  __shared__ __align__(16) double sb[kTileK][kTileN];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int64_t i0 = (int64_t)blockIdx.y * kTileM, j0 = (int64_t)blockIdx.x * kTileN;
  double acc[8][8] = {};
  // this thread's share of a slice: 4 elements of A and 4 of B
  double ra[4], rb[4];
  auto fetch = [&](int64_t k0) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = threadIdx.x + e * kThreads;      // 0 .. 1023
      const int kk_a = idx % kTileK, ii = idx / kTileK; // A: consecutive threads walk k (its unit stride when row-major)
      const int jj = idx % kTileN, kk_b = idx / kTileN; // B: consecutive threads walk j
      const int64_t i = i0 + ii, ka = k0 + kk_a, j = j0 + jj, kb = k0 + kk_b;
      ra[e] = (i < p.M && ka < p.K) ? p.a[i * p.a_r + ka * p.a_k] : 0.0;
      rb[e] = (j < p.N && kb < p.K) ? p.b[kb * p.b_k + j * p.b_c] : 0.0;
    }
  };
  auto stash = [&]() {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = threadIdx.x + e * kThreads;
      sa[idx % kTileK][idx / kTileK] = ra[e];
      sb[idx / kTileN][idx % kTileN] = rb[e];
    }
  };
  fetch(0);
  for (int64_t k0 = 0; k0 < p.K; k0 += kTileK) {
    stash();
    __syncthreads();
    if (k0 + kTileK < p.K)
      fetch(k0 + kTileK);
#pragma unroll
    for (int kk = 0; kk < kTileK; ++kk) {
      double av[8], bv[8];
      const double2 a0 = *reinterpret_cast<const double2 *>(&sa[kk][ty * 4]);
      const double2 a1 = *reinterpret_cast<const double2 *>(&sa[kk][ty * 4 + 2]);
      const double2 a2 = *reinterpret_cast<const double2 *>(&sa[kk][64 + ty * 4]);
      const double2 a3 = *reinterpret_cast<const double2 *>(&sa[kk][64 + ty * 4 + 2]);
      const double2 b0 = *reinterpret_cast<const double2 *>(&sb[kk][tx * 4]);
      const double2 b1 = *reinterpret_cast<const double2 *>(&sb[kk][tx * 4 + 2]);
      const double2 b2 = *reinterpret_cast<const double2 *>(&sb[kk][64 + tx * 4]);
      const double2 b3 = *reinterpret_cast<const double2 *>(&sb[kk][64 + tx * 4 + 2]);
      av[0] = a0.x, av[1] = a0.y, av[2] = a1.x, av[3] = a1.y, av[4] = a2.x, av[5] = a2.y, av[6] = a3.x, av[7] = a3.y;
      bv[0] = b0.x, bv[1] = b0.y, bv[2] = b1.x, bv[3] = b1.y, bv[4] = b2.x, bv[5] = b2.y, bv[6] = b3.x, bv[7] = b3.y;
#pragma unroll
      for (int r = 0; r < 8; ++r)
#pragma unroll
        for (int c = 0; c < 8; ++c)
          acc[r][c] = fma(av[r], bv[c], acc[r][c]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 8; ++r) {
    const int64_t i = i0 + (r < 4 ? 0 : 64) + ty * 4 + (r & 3);
    if (i >= p.M)
      continue;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const int64_t j = j0 + (c < 4 ? 0 : 64) + tx * 4 + (c & 3);
      if (j >= p.N)
        continue;
      double *dst = p.c + i * p.c_r + j * p.c_c;
      const double v = p.alpha * acc[r][c];
      *dst = p.beta == 0.0 ? v : fma(p.beta, *dst, v);
    }
  }
}

// The same product in 64 x 64 tiles (4 x 4 outputs per thread, 16 columns of K
// per step) for matrices with too few 128 x 128 tiles to fill the GPU.
constexpr int kSmallM = 64, kSmallN = 64, kSmallK = 16;

__global__ void __launch_bounds__(kThreads) nmb_gemm_f64_small(const GemmF64 p) {
  __shared__ double sa[kSmallK][kSmallM + 1];
  __shared__ double sb[kSmallK][kSmallN + 1];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4; // 16 x 16 threads, 4 x 4 outputs each
  const int64_t i0 = (int64_t)blockIdx.y * kSmallM, j0 = (int64_t)blockIdx.x * kSmallN;
  double acc[4][4] = {};
  for (int64_t k0 = 0; k0 < p.K; k0 += kSmallK) {
    // 64 x 16 elements of A and 16 x 64 of B: four of each per thread
    for (int e = threadIdx.x; e < kSmallM * kSmallK; e += kThreads) {
      const int kk = e % kSmallK, ii = e / kSmallK;
      const int64_t i = i0 + ii, k = k0 + kk;
      sa[kk][ii] = (i < p.M && k < p.K) ? p.a[i * p.a_r + k * p.a_k] : 0.0;
    }
    for (int e = threadIdx.x; e < kSmallN * kSmallK; e += kThreads) {
      const int jj = e % kSmallN, kk = e / kSmallN;
      const int64_t j = j0 + jj, k = k0 + kk;
      sb[kk][jj] = (j < p.N && k < p.K) ? p.b[k * p.b_k + j * p.b_c] : 0.0;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kSmallK; ++kk) {
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
  int64_t gy = (p.M + kTileM - 1) / kTileM, gx = (p.N + kTileN - 1) / kTileN;
  int sms = 148;
  cudaSetDevice(qv.device);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, qv.device);
  // 4096^3: 16.1 TFLOP/s with the large tiles against 10.5 with the small ones;
  // 1024^3 (64 large tiles on 148 multiprocessors): 7.6 against 10.6
  const bool small = gx * gy < (int64_t)sms;
  if (small) {
    gy = (p.M + kSmallM - 1) / kSmallM;
    gx = (p.N + kSmallN - 1) / kSmallN;
  }
  if (gy > 65535) {
    nmb::setError("mkl_gemm_float64_device: more than 65535 row tiles");
    return false;
  }
  const dim3 grid((unsigned)gx, (unsigned)gy);
  if (small)
    nmb_gemm_f64_small<<<grid, kThreads, 0, static_cast<cudaStream_t>(qv.stream)>>>(p);
  else
    nmb_gemm_f64<<<grid, kThreads, 0, static_cast<cudaStream_t>(qv.stream)>>>(p);
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
