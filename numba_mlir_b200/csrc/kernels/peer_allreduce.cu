// Stand-alone launches of the peer-memory all-reduce (peer_exchange.cuh): one
// block per GPU on the shard's own queue, for partial results that are not
// produced by one of the library's reduction kernels (those finish with the
// exchange themselves).
//
//   nmb_peer_allreduce_<op>_<type>   one array
//   nmb_peer_allreduce_multi         up to four arrays of different types and
//                                    operations behind ONE flag round trip
//                                    (the per-cluster sums and counts of a
//                                    k-means step)
#include "../gpu_common.h"
#include "peer_exchange.cuh"

namespace {

constexpr int kThreads = 1024;
namespace px = nmb::peer;

// type codes: 0 f32, 1 f64, 2 i32, 3 i64; op codes: 0 sum, 1 min, 2 max
template <typename F> __device__ __forceinline__ void with_type_op(int type, int op, F f) {
  auto typed = [&](auto zero) {
    if (op == 0)
      f(zero, px::OpSum());
    else if (op == 1)
      f(zero, px::OpMin());
    else
      f(zero, px::OpMax());
  };
  if (type == 0)
    typed(float(0));
  else if (type == 1)
    typed(double(0));
  else if (type == 2)
    typed(int32_t(0));
  else
    typed(int64_t(0));
}

__device__ __forceinline__ unsigned long long seg_bytes(int type, int64_t n) {
  const unsigned long long es = (type == 0 || type == 2) ? 4ull : 8ull;
  return ((unsigned long long)n * es + 15ull) & ~15ull;
}

} // namespace

// Launch: grid 1, block 1024.  `peers` holds `world` mailbox addresses as seen
// from this GPU (entry `rank` is this rank's own mailbox).
#define NMB_PEER_ALLREDUCE(op, OP, ty, T)                                                        \
  extern "C" __global__ void __launch_bounds__(kThreads)                                         \
      nmb_peer_allreduce_##op##_##ty(T *data, int64_t n, const unsigned long long *peers,       \
                                     int32_t rank, int32_t world, uint32_t *status) {            \
    px::allreduce_block<T>(data, n, peers, rank, world, status, OP());                          \
  }                                                                                              \
  NMB_REGISTER_KERNEL(nmb_peer_allreduce_##op##_##ty, 0);

#define NMB_PEER_ALLREDUCE_TYPES(op, OP)                                                         \
  NMB_PEER_ALLREDUCE(op, OP, f32, float)                                                         \
  NMB_PEER_ALLREDUCE(op, OP, f64, double)                                                        \
  NMB_PEER_ALLREDUCE(op, OP, i32, int32_t)                                                       \
  NMB_PEER_ALLREDUCE(op, OP, i64, int64_t)

NMB_PEER_ALLREDUCE_TYPES(sum, px::OpSum)
NMB_PEER_ALLREDUCE_TYPES(min, px::OpMin)
NMB_PEER_ALLREDUCE_TYPES(max, px::OpMax)

// Up to four segments (unused ones have n = 0); code = type + 4 * op.
extern "C" __global__ void __launch_bounds__(kThreads)
    nmb_peer_allreduce_multi(void *d0, int64_t n0, int32_t c0, void *d1, int64_t n1, int32_t c1, void *d2,
                             int64_t n2, int32_t c2, void *d3, int64_t n3, int32_t c3,
                             const unsigned long long *peers, int32_t rank, int32_t world,
                             uint32_t *status) {
  __shared__ px::Call call;
  void *data[4] = {d0, d1, d2, d3};
  const int64_t n[4] = {n0, n1, n2, n3};
  const int code[4] = {c0, c1, c2, c3};
  unsigned long long off[4], total = 0;
  bool codes_ok = true;
  for (int s = 0; s < 4; ++s) {
    off[s] = total;
    codes_ok = codes_ok && code[s] >= 0 && code[s] < 12 && n[s] >= 0;
    total += seg_bytes(code[s] & 3, n[s] > 0 ? n[s] : 0);
  }
  if (!codes_ok || !px::args_ok(rank, world, total)) {
    if (threadIdx.x == 0)
      atomicExch(status, (uint32_t)nmb::kStatusWaitTimeout);
    return;
  }
  px::begin(call, peers, rank, world);
  // everything is pushed before the first wait: the peers' waits overlap
  for (int s = 0; s < 4; ++s)
    if (n[s] > 0)
      with_type_op(code[s] & 3, code[s] >> 2, [&](auto zero, auto) {
        using T = decltype(zero);
        px::push(call, rank, world, static_cast<const T *>(data[s]), n[s], off[s]);
      });
  bool ok = true;
  for (int s = 0; s < 4 && ok; ++s)
    if (n[s] > 0)
      with_type_op(code[s] & 3, code[s] >> 2, [&](auto zero, auto op) {
        using T = decltype(zero);
        ok = px::pull(call, rank, world, static_cast<T *>(data[s]), n[s], off[s], op, status);
      });
  if (threadIdx.x == 0)
    px::end_call(call, rank);
}
NMB_REGISTER_KERNEL(nmb_peer_allreduce_multi, 0);
