// Column (first-axis) reductions: out[c] = reduce(a[:, c]).
// Launch: grid = (ceil(cols / ct), row_blocks) with ct the column-slab width
// (<= 16 KB of elements), 256 threads, about 444 CTAs in all; the scratch layout is
// described at reduce_cols_ws.  peers/rank/world: the mailbox table of the
// exchange between the GPUs' shards that ends the kernel (world <= 1: none).
#include "reduce_kernels.cuh"

#define COLS_KERNEL(kind, op, ty, R)                                                           \
  extern "C" __global__ void __launch_bounds__(nmb::red::kThreads, 3)                             \
      nmb_reduce_cols_##op##_##ty(const R::In *a, R::Out *out, void *partials,                 \
                                  uint32_t *counters, int64_t rows, int64_t cols,              \
                                  int64_t ct, int64_t fanin, uint32_t *status,                  \
                                  const unsigned long long *peers, int32_t rank,               \
                                  int32_t world) {                                             \
    extern __shared__ __align__(128) unsigned char nmb_smem[];                                 \
    nmb::red::reduce_cols_ws<R>(a, out, static_cast<R::Acc *>(partials), counters, rows,     \
                                  cols, ct, fanin, status, nmb_smem,                           \
                                  nmb::peer::Args{peers, rank, world});                        \
  }                                                                                            \
  NMB_REGISTER_KERNEL(nmb_reduce_cols_##op##_##ty, nmb::red::kSmemBytes);

NMB_RED_ALL_OPS(COLS_KERNEL, cols)
