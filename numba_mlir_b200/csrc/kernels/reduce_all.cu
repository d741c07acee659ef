// Full reductions out[0] = reduce(a[0:n]) and the layout-agnostic fallback.
// Launch (all): grid.x = G CTAs of 256 threads, span = per-CTA element count
// (multiple of 16384/sizeof(T)); scratch holds G accumulators and one zeroed
// counter; peers/rank/world: the exchange between the GPUs' shards that ends
// the kernel (world <= 1: none).  Launch (generic): mode 0 -> 32 threads per output, mode 1 -> one.
#include "reduce_kernels.cuh"

#define ALL_KERNEL(kind, op, ty, R)                                                            \
  extern "C" __global__ void __launch_bounds__(nmb::red::kThreads)                             \
      nmb_reduce_all_##op##_##ty(const R::In *a, R::Out *out, void *partials,                  \
                                 uint32_t *counter, int64_t n, int64_t span,                   \
                                 uint32_t *status, const unsigned long long *peers,            \
                                 int32_t rank, int32_t world) {                                \
    extern __shared__ __align__(128) unsigned char nmb_smem[];                                 \
    nmb::red::reduce_all_body<R>(a, out, static_cast<R::Acc *>(partials), counter, n, span,    \
                                 status, nmb_smem, nmb::peer::Args{peers, rank, world});       \
  }                                                                                            \
  NMB_REGISTER_KERNEL(nmb_reduce_all_##op##_##ty, nmb::red::kSmemBytes);                       \
  extern "C" __global__ void __launch_bounds__(nmb::red::kThreads)                             \
      nmb_reduce_generic_##op##_##ty(const R::In *a, R::Out *out, int64_t outer, int64_t K,    \
                                     int64_t inner, int64_t so, int64_t sk, int64_t si,        \
                                     int32_t mode) {                                           \
    nmb::red::reduce_generic_body<R>(a, out, outer, K, inner, so, sk, si, mode);               \
  }                                                                                            \
  NMB_REGISTER_KERNEL(nmb_reduce_generic_##op##_##ty, 0);

NMB_RED_ALL_OPS(ALL_KERNEL, all)
