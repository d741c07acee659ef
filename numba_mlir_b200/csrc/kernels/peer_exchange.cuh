// All-reduce of small partial results (at most 64 KB in all) across the GPUs
// of one box over peer memory, as a device routine run by ONE thread block:
// either the single block of the stand-alone kernels (peer_allreduce.cu) or
// the block of a reduction kernel that finishes last, so that a reduction over
// a sharded axis and its exchange are one launch.
//
// The exchange is latency bound (a few KB), so it is built to cost one one-way
// trip over NVLink and no fence: every rank PUSHES its partial into every
// peer's mailbox as 8-byte words {4 bytes of data, 4 bytes of the call's
// number}, and every rank polls its OWN mailbox, word by word, until the
// number it expects is there.  An aligned 8-byte store arrives whole, so a
// word whose number matches carries its data; nothing else orders the stores.
//
// Mailbox of one rank (in its own memory, mapped by the others):
//
//   bytes [0, 8)     the owner's call counter (read and written by the owner only)
//   bytes [256, ...) two slots; slot s holds, for every source rank r, a region
//                    of 128 KB (64 KB of payload as 16 Ki words of 8 bytes):
//                    offset 256 + (s * kMaxRanks + r) * 128 KB
//
// Every call advances the rank's own call counter; the new value `seq`
// (1, 2, ...; the same on every rank, since every rank takes part in every
// call) is the call's number, and keeping it on the device makes the launch
// identical from call to call, so a step that contains it can be recorded in a
// CUDA graph and replayed.  Call `seq` uses slot seq & 1 and tags its words
// with the low 32 bits of seq:
//   1. the rank stores its partial (one or several segments, packed at 16-byte
//      boundaries) as tagged words into its region of every peer's mailbox;
//   2. for each element it waits, with a bound, for the words of every peer in
//      its own mailbox and combines the ranks' values in rank order (so every
//      rank gets bit-identical results, floating-point sums included).
// A rank can only reach call seq + 2, which reuses the slot, after it has all of
// call seq + 1, and a peer sends its part of seq + 1 only after it has finished
// reading call seq: two slots are enough.  Tags differ between the two uses of
// a slot, so stale words are never taken for new ones (2^32 calls apart).
//
// The ranks are kernels on different GPUs.  They must not be emulated as
// separate launches on one GPU (nothing would guarantee that they run at the
// same time); a single-GPU test fills this rank's mailbox before the launch.
// If a peer never arrives the wait runs out, the status word is set, the
// segments are left untouched and the routine returns false.
//
// Plain peer stores and local volatile loads only: no multimem, no TMA on peer
// memory.
#pragma once

#include "bulk_pipe.cuh"

#include <cstdint>

namespace nmb {
namespace peer {

constexpr int kMaxRanks = 16;
constexpr unsigned long long kHeaderBytes = 256;
constexpr unsigned long long kPayloadBytes = 65536;            // most a call can carry
constexpr unsigned long long kRegionBytes = 2 * kPayloadBytes; // tagged words of one source rank
constexpr unsigned long long kMailboxBytes = kHeaderBytes + 2 * kMaxRanks * kRegionBytes;
constexpr long long kSpinLimit = 1ll << 22; // polls with back-off per thread: two seconds at the least

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

// What one block keeps in shared memory for a call.
struct Call {
  unsigned long long base[kMaxRanks];
  unsigned long long seq;
  int failed;
};

__device__ __forceinline__ bool args_ok(int rank, int world, unsigned long long bytes) {
  return world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world && bytes <= kPayloadBytes;
}

// Bytes a segment of n elements of T takes in the payload (16-byte granules).
template <typename T> __device__ __forceinline__ unsigned long long segment_bytes(int64_t n) {
  return ((unsigned long long)n * sizeof(T) + 15ull) & ~15ull;
}

// Step 0 (whole block): reads the mailbox table and the call number.  Several
// blocks of one kernel may take part in the same call, each with its own
// range of the payload: the counter is advanced once, by `end_call`, when all
// of them are done.
__device__ __forceinline__ void begin(Call &c, const unsigned long long *peers, int rank, int world) {
  const int tid = threadIdx.x;
  if (tid < world)
    c.base[tid] = peers[tid];
  if (tid == 0)
    c.failed = 0;
  __syncthreads();
  if (tid == 0)
    c.seq = *reinterpret_cast<volatile unsigned long long *>(c.base[rank]) + 1;
  __syncthreads();
}

// One thread, once per call, after the call's last block has finished.
__device__ __forceinline__ void end_call(const Call &c, int rank) {
  *reinterpret_cast<volatile unsigned long long *>(c.base[rank]) = c.seq;
}

// Address of the tagged words that source rank `src` leaves in the mailbox at
// `mailbox` for this call, from payload byte offset `off` on.
__device__ __forceinline__ unsigned long long *words_of(const Call &c, unsigned long long mailbox, int src,
                                                        unsigned long long off) {
  return reinterpret_cast<unsigned long long *>(mailbox + kHeaderBytes +
                                                ((c.seq & 1ull) * kMaxRanks + (unsigned)src) * kRegionBytes +
                                                2 * off);
}

template <typename T> union Words {
  T value;
  uint32_t w[sizeof(T) / 4];
};

// Step 1 (whole block): pushes one segment to every peer.  `data` may have been
// written by other blocks of the same kernel: it is read through L2.  Thread t
// sends the elements t, t + blockDim.x, ... -- the ones it combines in step 2.
template <typename T>
__device__ __forceinline__ void push(const Call &c, int rank, int world, const T *data, int64_t n,
                                     unsigned long long off) {
  constexpr int kW = sizeof(T) / 4;
  const uint32_t tag = (uint32_t)c.seq;
  for (int64_t e = threadIdx.x; e < n; e += blockDim.x) {
    const T v = __ldcg(data + e);
    Words<T> bits;
    bits.value = v;
    for (int p = 0; p < world; ++p) {
      if (p == rank)
        continue;
      unsigned long long *dst = words_of(c, c.base[p], rank, off) + e * kW;
#pragma unroll
      for (int k = 0; k < kW; ++k) {
        const unsigned long long word = ((unsigned long long)tag << 32) | bits.w[k];
        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst + k), "l"(word) : "memory");
      }
    }
  }
}

__device__ __forceinline__ unsigned long long load_word(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// Step 2 (whole block): data[e] = op over ranks, in rank order, of every
// rank's element e.  A thread takes kBatch elements at a time and has the
// words of all of them, from up to four peers, in flight at once; words that
// have not arrived yet are polled again.  Returns false (status word set,
// `data` as it was for the elements not yet combined) when a peer's words did
// not arrive in time.
template <typename T, typename Op>
__device__ __forceinline__ bool pull(Call &c, int rank, int world, T *data, int64_t n, unsigned long long off,
                                     Op op, uint32_t *status) {
  constexpr int kW = sizeof(T) / 4;
  constexpr int kBatch = 4, kPeers = 4;
  const uint32_t tag = (uint32_t)c.seq;
  long long budget = kSpinLimit;
  bool ok = true;
  for (int64_t e0 = threadIdx.x; e0 < n && ok; e0 += (int64_t)blockDim.x * kBatch) {
    T acc[kBatch];
    bool first = true;
    // ranks in order, four at a time; this rank's own values come from `data`
    for (int r0 = 0; r0 < world && ok; r0 += kPeers) {
      unsigned long long w[kPeers][kBatch][kW];
#pragma unroll
      for (int j = 0; j < kPeers; ++j)
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
          const int r = r0 + j;
          const int64_t e = e0 + (int64_t)u * blockDim.x;
          if (r < world && r != rank && e < n) {
            const unsigned long long *src = words_of(c, c.base[rank], r, off) + e * kW;
#pragma unroll
            for (int k = 0; k < kW; ++k)
              w[j][u][k] = load_word(src + k);
          }
        }
#pragma unroll
      for (int j = 0; j < kPeers; ++j)
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
          const int r = r0 + j;
          const int64_t e = e0 + (int64_t)u * blockDim.x;
          if (r >= world || e >= n)
            continue;
          T v;
          if (r == rank) {
            v = __ldcg(data + e);
          } else {
            const unsigned long long *src = words_of(c, c.base[rank], r, off) + e * kW;
            Words<T> bits;
#pragma unroll
            for (int k = 0; k < kW; ++k) {
              unsigned long long word = w[j][u][k];
              while ((uint32_t)(word >> 32) != tag && ok) {
                if (--budget < 0) {
                  ok = false;
                  break;
                }
                if (budget < kSpinLimit - 64)
                  __nanosleep(500);
                word = load_word(src + k);
              }
              bits.w[k] = (uint32_t)word;
            }
            v = bits.value;
          }
          acc[u] = (first && j == 0) ? v : op(acc[u], v);
        }
      first = false;
    }
    if (ok)
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        const int64_t e = e0 + (int64_t)u * blockDim.x;
        if (e < n)
          data[e] = acc[u];
      }
  }
  if (!ok)
    atomicExch(&c.failed, 1);
  __syncthreads();
  if (c.failed) {
    if (threadIdx.x == 0)
      atomicExch(status, (uint32_t)nmb::kStatusWaitTimeout);
    return false;
  }
  return true;
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
  push(call, rank, world, data, n, 0);
  const bool ok = pull(call, rank, world, data, n, 0, op, status);
  if (threadIdx.x == 0)
    end_call(call, rank);
  return ok;
}

// Arguments a reduction kernel takes to finish with the exchange; world <= 1
// means no exchange.
struct Args {
  const unsigned long long *peers;
  int rank, world;
};

} // namespace peer
} // namespace nmb
