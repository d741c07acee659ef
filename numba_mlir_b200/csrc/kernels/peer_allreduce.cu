// All-reduce of a small partial result (at most 64 KB) across the GPUs of one
// box over peer memory: no library collective, one launch of one block per GPU.
//
// The partials that span shards (a column-wise minimum, a full sum, the
// per-cluster sums and counts of a k-means step) are a few KB, so the exchange
// is pure latency; this kernel spends one flag round trip over NVLink instead
// of a collective library's launch and protocol.
//
// Every rank owns a mailbox in its own memory that the other ranks map:
//
//   bytes [0, 8)       flag of slot 0 (a 64-bit sequence number)
//   bytes [64, 72)     the owner's call counter (read and written by the owner only)
//   bytes [128, 136)   flag of slot 1
//   bytes [256, +64K)  payload of slot 0
//   then               payload of slot 1
//
// Every launch increments the rank's own call counter; the new value `seq`
// (1, 2, ...; the same on every rank, since every rank takes part in every
// call) is the call's number.  Keeping it on the device makes the launch
// identical from call to call, so a step that contains it can be recorded in a
// CUDA graph and replayed.  Call `seq` uses slot seq & 1:
//   1. the rank copies its partial into its own payload and then stores `seq`
//      into its own flag with release semantics at system scope;
//   2. it waits, with a bound, until every peer's flag of that slot reads `seq`;
//   3. it combines the payloads of all ranks in rank order (so every rank gets
//      bit-identical results, floating-point sums included) into `data`.
// A rank can only reach call seq + 2, which reuses the slot, after call seq + 1,
// and that one needs every peer's flag for seq + 1, which a peer stores only
// after its own call seq has finished reading: two slots are enough.
//
// The ranks are kernels on different GPUs.  They must not be emulated as
// separate launches on one GPU (nothing would guarantee that they run at the
// same time); a single-GPU test fills the peers' mailboxes before the launch.
// If a peer never arrives the wait runs out, the status word is set, `data` is
// left untouched and the launch returns.
#include "../gpu_common.h"
#include "bulk_pipe.cuh"

#include <cstdint>

namespace {

constexpr int kThreads = 1024;
constexpr int kMaxRanks = 16;
constexpr unsigned long long kFlagStride = 128;
constexpr unsigned long long kCounterOffset = 64;
constexpr unsigned long long kHeaderBytes = 256;
constexpr unsigned long long kSlotBytes = 65536;
constexpr int kSpinLimit = 1 << 22; // x (0.5 us of back-off + one flag read): two seconds at the least,
                                    // several when the flag is read over the link

struct OpSum {
  template <typename T> __device__ __forceinline__ T operator()(T a, T b) const { return a + b; }
};
// select(b < a, b, a) and select(a < b, b, a): the library's min and max
struct OpMin {
  template <typename T> __device__ __forceinline__ T operator()(T a, T b) const { return b < a ? b : a; }
};
struct OpMax {
  template <typename T> __device__ __forceinline__ T operator()(T a, T b) const { return a < b ? b : a; }
};

__device__ __forceinline__ unsigned long long load_flag(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void store_flag(unsigned long long *p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

template <typename T, typename Op>
__device__ __forceinline__ void peer_allreduce(T *data, int64_t n, const unsigned long long *peers,
                                               int rank, int world, uint32_t *status) {
  __shared__ unsigned long long base[kMaxRanks];
  __shared__ unsigned long long seq_shared;
  __shared__ int arrived;
  const int tid = threadIdx.x;
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world ||
      (unsigned long long)n * sizeof(T) > kSlotBytes) {
    if (tid == 0)
      atomicExch(status, (uint32_t)nmb::kStatusWaitTimeout);
    return;
  }
  if (tid < world)
    base[tid] = peers[tid];
  if (tid == 0)
    arrived = 1;
  __syncthreads();
  if (tid == 0) {
    unsigned long long *counter = reinterpret_cast<unsigned long long *>(base[rank] + kCounterOffset);
    seq_shared = *counter + 1;
    *counter = seq_shared;
  }
  __syncthreads();
  const unsigned long long seq = seq_shared;
  const unsigned long long slot = seq & 1ull;
  const unsigned long long payload = kHeaderBytes + slot * kSlotBytes;

  // 16-byte chunks when the partial allows it: a thread then has the loads of
  // four ranks in flight for each chunk, so the combine costs one trip over the
  // link per four ranks.
  constexpr int kPerChunk = 16 / sizeof(T);
  const bool chunked = (reinterpret_cast<unsigned long long>(data) & 15ull) == 0 && n % kPerChunk == 0;
  const int64_t nchunks = chunked ? n / kPerChunk : 0;

  // 1. publish this rank's partial
  T *mine = reinterpret_cast<T *>(base[rank] + payload);
  if (chunked) {
    for (int64_t c = tid; c < nchunks; c += kThreads)
      reinterpret_cast<uint4 *>(mine)[c] = reinterpret_cast<const uint4 *>(data)[c];
  } else {
    for (int64_t i = tid; i < n; i += kThreads)
      mine[i] = data[i];
  }
  __syncthreads();
  if (tid == 0) {
    // the block's stores above are ordered before this release through the barrier
    __threadfence_system();
    store_flag(reinterpret_cast<unsigned long long *>(base[rank] + slot * kFlagStride), seq);
  }

  // 2. one thread per peer waits for that peer's flag
  if (tid < world && tid != rank) {
    const unsigned long long *flag =
        reinterpret_cast<const unsigned long long *>(base[tid] + slot * kFlagStride);
    bool ok = false;
    for (int spin = 0; spin < kSpinLimit; ++spin) {
      if (load_flag(flag) == seq) {
        ok = true;
        break;
      }
      __nanosleep(spin < 64 ? 20 : 500);
    }
    if (!ok)
      atomicExch(&arrived, 0);
  }
  __syncthreads();
  if (!arrived) {
    if (tid == 0)
      atomicExch(status, (uint32_t)nmb::kStatusWaitTimeout);
    return;
  }

  // 3. combine in rank order; peers' payloads are read over the link, uncached
  const Op op;
  if (chunked) {
    for (int64_t c = tid; c < nchunks; c += kThreads) {
      // ranks in batches of four: four loads in flight, combined in rank order
      uint4 acc = __ldcv(reinterpret_cast<const uint4 *>(base[0] + payload) + c);
      for (int p0 = 1; p0 < world; p0 += 4) {
        uint4 part[4];
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (p0 + k < world)
            part[k] = __ldcv(reinterpret_cast<const uint4 *>(base[p0 + k] + payload) + c);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (p0 + k < world) {
            T *a = reinterpret_cast<T *>(&acc);
            const T *b = reinterpret_cast<const T *>(&part[k]);
#pragma unroll
            for (int l = 0; l < kPerChunk; ++l)
              a[l] = op(a[l], b[l]);
          }
      }
      reinterpret_cast<uint4 *>(data)[c] = acc;
    }
  } else {
    for (int64_t i = tid; i < n; i += kThreads) {
      T acc = __ldcv(reinterpret_cast<const T *>(base[0] + payload) + i);
      for (int p = 1; p < world; ++p)
        acc = op(acc, __ldcv(reinterpret_cast<const T *>(base[p] + payload) + i));
      data[i] = acc;
    }
  }
}

} // namespace

// Launch: grid 1, block 1024.  `peers` holds `world` mailbox addresses as seen
// from this GPU (entry `rank` is this rank's own mailbox).
#define NMB_PEER_ALLREDUCE(op, OP, ty, T)                                                        \
  extern "C" __global__ void __launch_bounds__(kThreads)                                         \
      nmb_peer_allreduce_##op##_##ty(T *data, int64_t n, const unsigned long long *peers,       \
                                     int32_t rank, int32_t world, uint32_t *status) {            \
    peer_allreduce<T, OP>(data, n, peers, rank, world, status);                                 \
  }                                                                                              \
  NMB_REGISTER_KERNEL(nmb_peer_allreduce_##op##_##ty, 0);

#define NMB_PEER_ALLREDUCE_TYPES(op, OP)                                                         \
  NMB_PEER_ALLREDUCE(op, OP, f32, float)                                                         \
  NMB_PEER_ALLREDUCE(op, OP, f64, double)                                                        \
  NMB_PEER_ALLREDUCE(op, OP, i32, int32_t)                                                       \
  NMB_PEER_ALLREDUCE(op, OP, i64, int64_t)

NMB_PEER_ALLREDUCE_TYPES(sum, OpSum)
NMB_PEER_ALLREDUCE_TYPES(min, OpMin)
NMB_PEER_ALLREDUCE_TYPES(max, OpMax)
