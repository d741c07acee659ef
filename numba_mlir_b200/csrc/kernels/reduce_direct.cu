// Row and full reductions (sum, prod, min, max) that read the array with plain
// 128-bit streaming loads, four per thread in flight, and reduce in registers:
// the one-pass reducers that the array front end generates around an
// elementwise chain (nmb::reduce_rows_fused / reduce_all_fused in
// nmb_device.cuh), instantiated here ahead of time for the chain "the array
// itself".  On B200 they measured faster than the shared-memory ring of TMA
// bulk copies (reduce_ws.cuh) for these two shapes -- float32 (16384, 4096)
// sum(axis=1) 41.4 us against 43.9 us, 2^28 int32 full sum 152.3 us against
// 162.9 us -- so the host dispatch uses them, and a warp-per-row argmin/argmax
// built the same way; column reductions (a direct-load column kernel took
// 61-65 us against the ring's 47 us on the same matrix), and argmin/argmax over a
// few long rows, stay on the ring.  Same semantics as there: sum/prod accumulate
// in int64 for int32 input and in the array type otherwise, min/max are
// select(x < m), NaNs never win, partials merged in index order.
//
// A full reduction over one GPU's shard finishes with the exchange between
// the GPUs (peer_exchange.cuh) in the block that wrote the result.
#include "../gpu_common.h"
#include "nmb_device.cuh"
#include "peer_exchange.cuh"

namespace {

constexpr int kBlock = 256;
constexpr int kUnroll = 4;

template <typename T> struct PlainChain {
  const T *__restrict__ in0;
  template <int V> struct In {
    nmb::Vec<T, V> in0;
  };
  template <int V> struct Out {
    nmb::Vec<T, V> out0;
  };
  template <int V> __device__ __forceinline__ void load(int64_t i, In<V> &r) const {
    r.in0 = nmb::load_stream<T, V>(in0 + i);
  }
  template <int V> __device__ __forceinline__ void compute(const In<V> &r, Out<V> &o) const { o.out0 = r.in0; }
  template <typename A> __device__ __forceinline__ A post(A v) const { return v; }
};

template <typename T> struct Wide { using type = T; };
template <> struct Wide<int32_t> { using type = int64_t; };

struct SumTag {
  using Op = nmb::OpAdd;
  template <typename T> using Acc = typename Wide<T>::type;
  template <typename A> static __device__ __forceinline__ A identity() { return A(0); }
};
struct ProdTag {
  using Op = nmb::OpMul;
  template <typename T> using Acc = typename Wide<T>::type;
  template <typename A> static __device__ __forceinline__ A identity() { return A(1); }
};
struct MinTag {
  using Op = nmb::OpMin;
  template <typename T> using Acc = T;
  template <typename A> static __device__ __forceinline__ A identity() { return nmb::neutral_min<A>(); }
};
struct MaxTag {
  using Op = nmb::OpMax;
  template <typename T> using Acc = T;
  template <typename A> static __device__ __forceinline__ A identity() { return nmb::neutral_max<A>(); }
};

// out[r] = reduce(a[r, :]); cols % (16 / sizeof(T)) == 0, a 16-byte aligned.
template <typename Tag, typename T, bool BLOCK_ROW>
__device__ __forceinline__ void rows_direct(const T *a, typename Tag::template Acc<T> *out, int64_t rows,
                                            int64_t cols) {
  using A = typename Tag::template Acc<T>;
  constexpr int V = 16 / sizeof(T);
  __shared__ A scratch[32];
  PlainChain<T> chain{a};
  nmb::reduce_rows_fused<kBlock, V, kUnroll, BLOCK_ROW>(chain, rows, cols, out, typename Tag::Op(),
                                                        Tag::template identity<A>(), scratch);
}

// out[0] = reduce(a[0:n]); a 16-byte aligned.
template <typename Tag, typename T>
__device__ __forceinline__ void all_direct(const T *a, typename Tag::template Acc<T> *out, void *partials,
                                           uint32_t *counter, int64_t n, uint32_t *status,
                                           const nmb::peer::Args px) {
  using A = typename Tag::template Acc<T>;
  constexpr int V = 16 / sizeof(T);
  __shared__ A scratch[32];
  PlainChain<T> chain{a};
  const bool wrote = nmb::reduce_all_fused<kBlock, V, kUnroll>(chain, n, out, static_cast<A *>(partials), counter,
                                                               typename Tag::Op(), Tag::template identity<A>(),
                                                               scratch);
  if (wrote && px.world > 1) {
    __syncthreads();
    nmb::peer::allreduce_block<A>(out, 1, px.peers, px.rank, px.world, status, typename Tag::Op());
  }
}

// out[r] = index of the first minimum (MIN) or maximum of a[r, :], one warp per
// row.  A lane visits its elements in increasing index order, so a strict
// comparison keeps the first occurrence; between lanes the lower index wins
// ties.  NaNs never compare true and are passed over, as in the ring kernels;
// a row in which nothing beats the identity gives index 0.
template <typename T, bool MIN>
__device__ __forceinline__ void rows_arg_direct(const T *__restrict__ a, int64_t *__restrict__ out,
                                                int64_t rows, int64_t cols) {
  constexpr int V = 16 / sizeof(T);
  constexpr int64_t kNone = 0x7fffffffffffffffll;
  const int lane = threadIdx.x & 31;
  const int64_t first = (int64_t)blockIdx.x * (kBlock / 32) + (threadIdx.x >> 5);
  const int64_t step = (int64_t)gridDim.x * (kBlock / 32);
  constexpr int64_t span = 32 * V * kUnroll;
  auto beats = [](T x, T v) { return MIN ? x < v : v < x; };
  for (int64_t r = first; r < rows; r += step) {
    const T *row = a + r * cols;
    T bv = MIN ? nmb::neutral_min<T>() : nmb::neutral_max<T>();
    int64_t bi = kNone;
    int64_t k0 = 0;
    for (; k0 + span <= cols; k0 += span) {
      nmb::Vec<T, V> x[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
        x[u] = nmb::load_stream<T, V>(row + k0 + (u * 32 + lane) * V);
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
#pragma unroll
        for (int l = 0; l < V; ++l)
          if (beats(x[u].v[l], bv)) {
            bv = x[u].v[l];
            bi = k0 + (u * 32 + lane) * V + l;
          }
    }
    for (int64_t k = k0 + lane * V; k < cols; k += 32 * V) {
      const nmb::Vec<T, V> x = nmb::load_stream<T, V>(row + k);
#pragma unroll
      for (int l = 0; l < V; ++l)
        if (beats(x.v[l], bv)) {
          bv = x.v[l];
          bi = k + l;
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const T ov = __shfl_xor_sync(0xffffffffu, bv, off);
      const int64_t oi = __shfl_xor_sync(0xffffffffu, bi, off);
      if (beats(ov, bv) || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    if (lane == 0)
      out[r] = bi == kNone ? 0 : bi;
  }
}

} // namespace

// Launch (rows): grid.x blocks of 256 threads; a row belongs to one warp, or to
// the whole block in the `_blockrow` variant (few long rows).
// Launch (all): grid.x blocks of 256 threads taking tiles of 256 * (16 /
// sizeof(T)) * 4 elements round robin; scratch holds grid.x accumulators and one
// zeroed counter; peers/rank/world: the exchange that ends the kernel
// (world <= 1: none).
// Resident blocks per multiprocessor the row kernels are compiled for: eight
// for float32 (32 registers hold everything), six for the types with 64-bit
// values or accumulators.
#define NMB_ROWS_RESIDENT_f32 8
#define NMB_ROWS_RESIDENT_f64 6
#define NMB_ROWS_RESIDENT_i32 6
#define NMB_ROWS_RESIDENT_i64 6

#define NMB_DIRECT(op, TAG, ty, T)                                                                         \
  extern "C" __global__ void __launch_bounds__(kBlock, NMB_ROWS_RESIDENT_##ty)                               \
      nmb_reduce_rows_direct_##op##_##ty(const T *a, TAG::Acc<T> *out, int64_t rows, int64_t cols) {       \
    rows_direct<TAG, T, false>(a, out, rows, cols);                                                        \
  }                                                                                                        \
  NMB_REGISTER_KERNEL(nmb_reduce_rows_direct_##op##_##ty, 0);                                              \
  extern "C" __global__ void __launch_bounds__(kBlock, NMB_ROWS_RESIDENT_##ty)                               \
      nmb_reduce_rows_direct_blockrow_##op##_##ty(const T *a, TAG::Acc<T> *out, int64_t rows,              \
                                                  int64_t cols) {                                          \
    rows_direct<TAG, T, true>(a, out, rows, cols);                                                         \
  }                                                                                                        \
  NMB_REGISTER_KERNEL(nmb_reduce_rows_direct_blockrow_##op##_##ty, 0);                                     \
  extern "C" __global__ void __launch_bounds__(kBlock, 6)                                                   \
      nmb_reduce_all_direct_##op##_##ty(const T *a, TAG::Acc<T> *out, void *partials, uint32_t *counter,   \
                                        int64_t n, uint32_t *status, const unsigned long long *peers,      \
                                        int32_t rank, int32_t world) {                                     \
    all_direct<TAG, T>(a, out, partials, counter, n, status, nmb::peer::Args{peers, rank, world});         \
  }                                                                                                        \
  NMB_REGISTER_KERNEL(nmb_reduce_all_direct_##op##_##ty, 0);

#define NMB_DIRECT_TYPES(op, TAG)                                                                          \
  NMB_DIRECT(op, TAG, f32, float)                                                                          \
  NMB_DIRECT(op, TAG, f64, double)                                                                         \
  NMB_DIRECT(op, TAG, i32, int32_t)                                                                        \
  NMB_DIRECT(op, TAG, i64, int64_t)

NMB_DIRECT_TYPES(sum, SumTag)
NMB_DIRECT_TYPES(prod, ProdTag)
NMB_DIRECT_TYPES(min, MinTag)
NMB_DIRECT_TYPES(max, MaxTag)

#define NMB_DIRECT_ARG(op, MIN, ty, T)                                                                     \
  extern "C" __global__ void __launch_bounds__(kBlock, 6)                                                  \
      nmb_reduce_rows_direct_##op##_##ty(const T *a, int64_t *out, int64_t rows, int64_t cols) {           \
    rows_arg_direct<T, MIN>(a, out, rows, cols);                                                           \
  }                                                                                                        \
  NMB_REGISTER_KERNEL(nmb_reduce_rows_direct_##op##_##ty, 0);

#define NMB_DIRECT_ARG_TYPES(op, MIN)                                                                      \
  NMB_DIRECT_ARG(op, MIN, f32, float)                                                                      \
  NMB_DIRECT_ARG(op, MIN, f64, double)                                                                     \
  NMB_DIRECT_ARG(op, MIN, i32, int32_t)                                                                    \
  NMB_DIRECT_ARG(op, MIN, i64, int64_t)

NMB_DIRECT_ARG_TYPES(argmin, true)
NMB_DIRECT_ARG_TYPES(argmax, false)
