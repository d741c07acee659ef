// Dense-contraction library entry points (placeholder translation unit: the
// tcgen05 kernels land here).
#include "gpu_common.h"

#define GPUX_EXPORT extern "C" __attribute__((visibility("default")))

GPUX_EXPORT void _mlir_ciface_mkl_gemm_float32_device(void *, const GPUXMemref2f *,
                                                      const GPUXMemref2f *, float,
                                                      float, GPUXMemref2f *) {
  nmb::setError("mkl_gemm_float32_device: not built yet");
}
GPUX_EXPORT void mkl_gemm_float32_device(void *q, const GPUXMemref2f *a,
                                         const GPUXMemref2f *b, float alpha,
                                         float beta, GPUXMemref2f *c) {
  _mlir_ciface_mkl_gemm_float32_device(q, a, b, alpha, beta, c);
}
GPUX_EXPORT void *_mlir_ciface_nmb_pairwise_distance_float32_device(
    void *, const GPUXMemref2f *, const GPUXMemref2f *, GPUXMemref2f *) {
  nmb::setError("nmb_pairwise_distance_float32_device: not built yet");
  return nullptr;
}
