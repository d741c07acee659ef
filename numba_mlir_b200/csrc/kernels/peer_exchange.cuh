// All-reduce of small partial results (at most 64 KB in all) across the GPUs
// of one box over peer memory, as a device routine run by ONE thread block:
// either the single block of the stand-alone kernels (peer_allreduce.cu) or
// the block of a reduction kernel that finishes last, so that a reduction over
// a sharded axis and its exchange are one launch.
//
// Every rank owns a mailbox in its own memory that the other ranks map:
//
//   bytes [0, 8)       flag of slot 0 (a 64-bit sequence number)
//   bytes [64, 72)     the owner's call counter (read and written by the owner only)
//   bytes [128, 136)   flag of slot 1
//   bytes [256, +64K)  payload of slot 0
//   then               payload of slot 1
//
// Every call increments the rank's own call counter; the new value `seq`
// (1, 2, ...; the same on every rank, since every rank takes part in every
// call) is the call's number.  Keeping it on the device makes the launch
// identical from call to call, so a step that contains it can be recorded in a
// CUDA graph and replayed.  Call `seq` uses slot seq & 1:
//   1. the rank copies its partials (one or several segments, packed at
//      16-byte boundaries) into its own payload and then stores `seq` into its
//      own flag with release semantics at system scope;
//   2. it waits, with a bound, until every peer's flag of that slot reads `seq`;
//   3. it combines the payloads of all ranks in rank order (so every rank gets
//      bit-identical results, floating-point sums included) into the segments.
// A rank can only reach call seq + 2, which reuses the slot, after call seq + 1,
// and that one needs every peer's flag for seq + 1, which a peer stores only
// after its own call seq has finished reading: two slots are enough.
//
// The ranks are kernels on different GPUs.  They must not be emulated as
// separate launches on one GPU (nothing would guarantee that they run at the
// same time); a single-GPU test fills the peers' mailboxes before the launch.
// If a peer never arrives the wait runs out, the status word is set, the
// segments are left untouched and the routine returns false.
//
// Plain peer loads and stores only (ld.acquire.sys / st.release.sys for the
// flags): no multimem, no TMA on peer memory.
#pragma once

#include "bulk_pipe.cuh"

#include <cstdint>

namespace nmb {
namespace peer {

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
struct OpProd {
  template <typename T> __device__ __forceinline__ T operator()(T a, T b) const { return a * b; }
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

// What one block keeps in shared memory for a call.
struct Call {
  unsigned long long base[kMaxRanks];
  unsigned long long seq;
  int arrived;
};

__device__ __forceinline__ bool args_ok(int rank, int world, unsigned long long bytes) {
  return world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world && bytes <= kSlotBytes;
}

// Bytes a segment of n elements of T takes in the payload (16-byte granules).
template <typename T> __device__ __forceinline__ unsigned long long segment_bytes(int64_t n) {
  return ((unsigned long long)n * sizeof(T) + 15ull) & ~15ull;
}

// Step 0 (whole block): reads the mailbox table and draws the call number.
__device__ __forceinline__ void begin(Call &c, const unsigned long long *peers, int rank, int world) {
  const int tid = threadIdx.x;
  if (tid < world)
    c.base[tid] = peers[tid];
  if (tid == 0)
    c.arrived = 1;
  __syncthreads();
  if (tid == 0) {
    unsigned long long *counter = reinterpret_cast<unsigned long long *>(c.base[rank] + kCounterOffset);
    c.seq = *counter + 1;
    *counter = c.seq;
  }
  __syncthreads();
}

__device__ __forceinline__ unsigned long long payload_of(const Call &c) {
  return kHeaderBytes + (c.seq & 1ull) * kSlotBytes;
}

template <typename T> __device__ __forceinline__ bool chunked(const T *data, int64_t n) {
  return (reinterpret_cast<unsigned long long>(data) & 15ull) == 0 && n % (16 / (int)sizeof(T)) == 0;
}

// Step 1 (whole block): copies one segment into this rank's payload at byte
// offset `off`.  `data` may have been written by other blocks of the same
// kernel: it is read through L2.
template <typename T>
__device__ __forceinline__ void publish(const Call &c, int rank, const T *data, int64_t n,
                                        unsigned long long off) {
  T *mine = reinterpret_cast<T *>(c.base[rank] + payload_of(c) + off);
  if (chunked(data, n)) {
    const int64_t nchunks = n / (16 / (int)sizeof(T));
    for (int64_t k = threadIdx.x; k < nchunks; k += blockDim.x)
      reinterpret_cast<uint4 *>(mine)[k] = __ldcg(reinterpret_cast<const uint4 *>(data) + k);
  } else {
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x)
      mine[i] = __ldcg(data + i);
  }
}

// Step 2 (whole block): raises this rank's flag, then one thread per peer waits
// for that peer's flag.  Returns false (status word set) when a wait ran out.
__device__ __forceinline__ bool signal_and_wait(Call &c, int rank, int world, uint32_t *status) {
  const int tid = threadIdx.x;
  const unsigned long long slot = c.seq & 1ull;
  __syncthreads();
  if (tid == 0) {
    // the block's stores above are ordered before this release through the barrier
    __threadfence_system();
    store_flag(reinterpret_cast<unsigned long long *>(c.base[rank] + slot * kFlagStride), c.seq);
  }
  if (tid < world && tid != rank) {
    const unsigned long long *flag =
        reinterpret_cast<const unsigned long long *>(c.base[tid] + slot * kFlagStride);
    bool ok = false;
    for (int spin = 0; spin < kSpinLimit; ++spin) {
      if (load_flag(flag) == c.seq) {
        ok = true;
        break;
      }
      __nanosleep(spin < 64 ? 20 : 500);
    }
    if (!ok)
      atomicExch(&c.arrived, 0);
  }
  __syncthreads();
  if (!c.arrived) {
    if (tid == 0)
      atomicExch(status, (uint32_t)nmb::kStatusWaitTimeout);
    return false;
  }
  return true;
}

// Step 3 (whole block): data[i] = op over ranks, in rank order, of the
// segment at payload offset `off`; peers' payloads are read over the link,
// uncached.
template <typename T, typename Op>
__device__ __forceinline__ void combine(const Call &c, int world, T *data, int64_t n,
                                        unsigned long long off, Op op) {
  const unsigned long long payload = payload_of(c) + off;
  constexpr int kPerChunk = 16 / sizeof(T);
  if (chunked(data, n)) {
    const int64_t nchunks = n / kPerChunk;
    for (int64_t k = threadIdx.x; k < nchunks; k += blockDim.x) {
      // ranks in batches of four: four loads in flight, combined in rank order
      uint4 acc = __ldcv(reinterpret_cast<const uint4 *>(c.base[0] + payload) + k);
      for (int p0 = 1; p0 < world; p0 += 4) {
        uint4 part[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (p0 + j < world)
            part[j] = __ldcv(reinterpret_cast<const uint4 *>(c.base[p0 + j] + payload) + k);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (p0 + j < world) {
            T *a = reinterpret_cast<T *>(&acc);
            const T *b = reinterpret_cast<const T *>(&part[j]);
#pragma unroll
            for (int l = 0; l < kPerChunk; ++l)
              a[l] = op(a[l], b[l]);
          }
      }
      reinterpret_cast<uint4 *>(data)[k] = acc;
    }
  } else {
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
      T acc = __ldcv(reinterpret_cast<const T *>(c.base[0] + payload) + i);
      for (int p = 1; p < world; ++p)
        acc = op(acc, __ldcv(reinterpret_cast<const T *>(c.base[p] + payload) + i));
      data[i] = acc;
    }
  }
}

// The whole call for one segment.  Every thread of the block must call it.
template <typename T, typename Op>
__device__ __forceinline__ bool allreduce_block(T *data, int64_t n, const unsigned long long *peers, int rank,
                                                int world, uint32_t *status, Op op) {
  __shared__ Call call;
  if (!args_ok(rank, world, (unsigned long long)n * sizeof(T))) {
    if (threadIdx.x == 0)
      atomicExch(status, (uint32_t)nmb::kStatusWaitTimeout);
    return false;
  }
  begin(call, peers, rank, world);
  publish(call, rank, data, n, 0);
  if (!signal_and_wait(call, rank, world, status))
    return false;
  combine(call, world, data, n, 0, op);
  return true;
}

// Arguments a reduction kernel takes to finish with the exchange; world <= 1
// means no exchange.
struct Args {
  const unsigned long long *peers;
  int rank, world;
};

} // namespace peer
} // namespace nmb
