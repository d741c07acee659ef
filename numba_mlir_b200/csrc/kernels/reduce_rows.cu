// Row (last-axis) reductions: out[r] = reduce(a[r, :]).
// Launch: grid.x = up to 444 CTAs of 256 threads (three per SM).
#include "reduce_kernels.cuh"

#define ROWS_KERNEL(kind, op, ty, R)                                                           \
  extern "C" __global__ void __launch_bounds__(nmb::red::kThreads, 3)                             \
      nmb_reduce_rows_##op##_##ty(const R::In *a, R::Out *out, int64_t rows, int64_t cols,     \
                                  uint32_t *status) {                                          \
    extern __shared__ __align__(128) unsigned char nmb_smem[];                                 \
    nmb::red::reduce_rows_ws<R>(a, out, rows, cols, status, nmb_smem);                       \
  }                                                                                            \
  NMB_REGISTER_KERNEL(nmb_reduce_rows_##op##_##ty, nmb::red::kSmemBytes);

NMB_RED_ALL_OPS(ROWS_KERNEL, rows)
