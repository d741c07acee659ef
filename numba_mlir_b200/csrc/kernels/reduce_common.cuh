// Reducers and kernel bodies for axis and full reductions.
//
// Semantics follow the reference's _array_reduce
// (numba_mlir/numba_mlir/mlir/numpy/funcs.py:163-214): sum/prod accumulate in
// int64 for every integer dtype and in the array dtype for floats; min/max are
// select(a < b, a, b) with +-inf / integer limits as identity (:278-295);
// argmin/argmax use the (value, index) pair combiner that keeps the lower index
// on ties (numba_mlir/mlir/builtin/funcs.py:118-138).  NaNs are not ordered by
// `<` and are therefore ignored, as in the reference's select.
//
// Data movement: the reduced matrix is streamed through shared memory in 16 KB
// tiles by the TMA bulk-copy engine (4-stage mbarrier ring per CTA), reduced
// from shared memory with 128-bit reads, then combined with warp shuffles.
// Cross-CTA combination (column and full reductions) goes through partials in
// scratch memory and ticket counters:
// the CTA that draws the last ticket merges the partials in index order, so
// results do not depend on scheduling.
#pragma once

#include "bulk_pipe.cuh"
#include "peer_exchange.cuh"

#include <type_traits>

namespace nmb {
namespace red {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kTileBytes = 16384;
constexpr int kStages = 4;
constexpr int kSmemBytes = kStages * kTileBytes + 64 + 32 * 16;

template <typename T> struct Limits;
template <> struct Limits<float> {
  static __device__ __forceinline__ float lowest() { return -__int_as_float(0x7f800000); }
  static __device__ __forceinline__ float highest() { return __int_as_float(0x7f800000); }
};
template <> struct Limits<double> {
  static __device__ __forceinline__ double lowest() { return -__longlong_as_double(0x7ff0000000000000ll); }
  static __device__ __forceinline__ double highest() { return __longlong_as_double(0x7ff0000000000000ll); }
};
template <> struct Limits<int32_t> {
  static __device__ __forceinline__ int32_t lowest() { return (int32_t)0x80000000; }
  static __device__ __forceinline__ int32_t highest() { return 0x7fffffff; }
};
template <> struct Limits<int64_t> {
  static __device__ __forceinline__ int64_t lowest() { return (int64_t)0x8000000000000000ll; }
  static __device__ __forceinline__ int64_t highest() { return 0x7fffffffffffffffll; }
};

// Atomic minimum and maximum in global memory.  Floats go through their bit
// patterns: values with a clear sign bit order like signed integers, values with
// the sign bit set in reverse like unsigned integers, and every pattern of the
// second kind is below every pattern of the first, so one integer atomic per
// call keeps the order (-0.0 counts as below +0.0).  NaNs must not be passed.
__device__ __forceinline__ void atomic_min(int32_t *p, int32_t v) { atomicMin(p, v); }
__device__ __forceinline__ void atomic_max(int32_t *p, int32_t v) { atomicMax(p, v); }
__device__ __forceinline__ void atomic_min(int64_t *p, int64_t v) {
  atomicMin(reinterpret_cast<long long *>(p), (long long)v);
}
__device__ __forceinline__ void atomic_max(int64_t *p, int64_t v) {
  atomicMax(reinterpret_cast<long long *>(p), (long long)v);
}
__device__ __forceinline__ void atomic_min(float *p, float v) {
  const int b = __float_as_int(v);
  if (b >= 0)
    atomicMin(reinterpret_cast<int *>(p), b);
  else
    atomicMax(reinterpret_cast<unsigned int *>(p), (unsigned int)b);
}
__device__ __forceinline__ void atomic_max(float *p, float v) {
  const int b = __float_as_int(v);
  if (b >= 0)
    atomicMax(reinterpret_cast<int *>(p), b);
  else
    atomicMin(reinterpret_cast<unsigned int *>(p), (unsigned int)b);
}
__device__ __forceinline__ void atomic_min(double *p, double v) {
  const long long b = __double_as_longlong(v);
  if (b >= 0)
    atomicMin(reinterpret_cast<long long *>(p), b);
  else
    atomicMax(reinterpret_cast<unsigned long long *>(p), (unsigned long long)b);
}
__device__ __forceinline__ void atomic_max(double *p, double v) {
  const long long b = __double_as_longlong(v);
  if (b >= 0)
    atomicMax(reinterpret_cast<long long *>(p), b);
  else
    atomicMin(reinterpret_cast<unsigned long long *>(p), (unsigned long long)b);
}

template <typename T> struct WideAcc { using type = T; };
template <> struct WideAcc<int32_t> { using type = int64_t; };

template <typename T> struct SumR {
  using In = T;
  using Acc = typename WideAcc<T>::type;
  using Out = Acc;
  static __device__ __forceinline__ Acc identity() { return Acc(0); }
  static __device__ __forceinline__ void acc(Acc &a, T x, int64_t) { a += (Acc)x; }
  static __device__ __forceinline__ Acc merge(Acc a, Acc b) { return a + b; }
  static __device__ __forceinline__ Acc shfl(Acc a, int off) { return __shfl_xor_sync(0xffffffffu, a, off); }
  static __device__ __forceinline__ Out fin(Acc a) { return a; }
  // Hot-loop accumulator: position k counts the thread's visits in increasing
  // index order; only index-carrying reducers need it.
  using Fast = Acc;
  static constexpr bool kTwoPass = false;
  static constexpr bool kAtomicCols = false;
  static __device__ __forceinline__ Fast fast_identity() { return identity(); }
  static __device__ __forceinline__ void fast_acc(Fast &a, T x, int) { acc(a, x, 0); }
  template <typename F> static __device__ __forceinline__ Acc widen_fn(Fast f, F) { return f; }
};
template <typename T> struct ProdR {
  using In = T;
  using Acc = typename WideAcc<T>::type;
  using Out = Acc;
  static __device__ __forceinline__ Acc identity() { return Acc(1); }
  static __device__ __forceinline__ void acc(Acc &a, T x, int64_t) { a *= (Acc)x; }
  static __device__ __forceinline__ Acc merge(Acc a, Acc b) { return a * b; }
  static __device__ __forceinline__ Acc shfl(Acc a, int off) { return __shfl_xor_sync(0xffffffffu, a, off); }
  static __device__ __forceinline__ Out fin(Acc a) { return a; }
  // Hot-loop accumulator: position k counts the thread's visits in increasing
  // index order; only index-carrying reducers need it.
  using Fast = Acc;
  static constexpr bool kTwoPass = false;
  static constexpr bool kAtomicCols = false;
  static __device__ __forceinline__ Fast fast_identity() { return identity(); }
  static __device__ __forceinline__ void fast_acc(Fast &a, T x, int) { acc(a, x, 0); }
  template <typename F> static __device__ __forceinline__ Acc widen_fn(Fast f, F) { return f; }
};
template <typename T> struct MinR {
  using In = T;
  using Acc = T;
  using Out = T;
  static __device__ __forceinline__ Acc identity() { return Limits<T>::highest(); }
  static __device__ __forceinline__ void acc(Acc &a, T x, int64_t) { a = x < a ? x : a; }
  static __device__ __forceinline__ Acc merge(Acc a, Acc b) { return b < a ? b : a; }
  static __device__ __forceinline__ Acc shfl(Acc a, int off) { return __shfl_xor_sync(0xffffffffu, a, off); }
  static __device__ __forceinline__ Out fin(Acc a) { return a; }
  // Hot-loop accumulator: position k counts the thread's visits in increasing
  // index order; only index-carrying reducers need it.
  using Fast = Acc;
  static constexpr bool kTwoPass = false;
  // Column reductions of different row blocks meet in `out` through atomics
  // (any order gives the same value) instead of a merge tree.
  static constexpr bool kAtomicCols = true;
  static __device__ __forceinline__ void atomic_merge(Out *p, Acc v) { atomic_min(p, v); }
  static __device__ __forceinline__ Fast fast_identity() { return identity(); }
  static __device__ __forceinline__ void fast_acc(Fast &a, T x, int) { acc(a, x, 0); }
  template <typename F> static __device__ __forceinline__ Acc widen_fn(Fast f, F) { return f; }
};
template <typename T> struct MaxR {
  using In = T;
  using Acc = T;
  using Out = T;
  static __device__ __forceinline__ Acc identity() { return Limits<T>::lowest(); }
  static __device__ __forceinline__ void acc(Acc &a, T x, int64_t) { a = a < x ? x : a; }
  static __device__ __forceinline__ Acc merge(Acc a, Acc b) { return a < b ? b : a; }
  static __device__ __forceinline__ Acc shfl(Acc a, int off) { return __shfl_xor_sync(0xffffffffu, a, off); }
  static __device__ __forceinline__ Out fin(Acc a) { return a; }
  // Hot-loop accumulator: position k counts the thread's visits in increasing
  // index order; only index-carrying reducers need it.
  using Fast = Acc;
  static constexpr bool kTwoPass = false;
  // Column reductions of different row blocks meet in `out` through atomics
  // (any order gives the same value) instead of a merge tree.
  static constexpr bool kAtomicCols = true;
  static __device__ __forceinline__ void atomic_merge(Out *p, Acc v) { atomic_max(p, v); }
  static __device__ __forceinline__ Fast fast_identity() { return identity(); }
  static __device__ __forceinline__ void fast_acc(Fast &a, T x, int) { acc(a, x, 0); }
  template <typename F> static __device__ __forceinline__ Acc widen_fn(Fast f, F) { return f; }
};

template <typename T> struct alignas(16) ValIdx {
  T v;
  int64_t i;
};
// MIN = true: argmin, false: argmax.  The lower index wins ties whatever the
// merge order, so the result is NumPy's first occurrence.
template <typename T, bool MIN> struct ArgR {
  using In = T;
  using Acc = ValIdx<T>;
  using Out = int64_t;
  static __device__ __forceinline__ Acc identity() {
    return Acc{MIN ? Limits<T>::highest() : Limits<T>::lowest(), 0x7fffffffffffffffll};
  }
  static __device__ __forceinline__ bool better(T xv, int64_t xi, T av, int64_t ai) {
    return MIN ? (xv < av || (xv == av && xi < ai)) : (av < xv || (xv == av && xi < ai));
  }
  static __device__ __forceinline__ void acc(Acc &a, T x, int64_t idx) {
    if (better(x, idx, a.v, a.i)) {
      a.v = x;
      a.i = idx;
    }
  }
  static __device__ __forceinline__ Acc merge(Acc a, Acc b) { return better(b.v, b.i, a.v, a.i) ? b : a; }
  static __device__ __forceinline__ Acc shfl(Acc a, int off) {
    Acc r;
    r.v = __shfl_xor_sync(0xffffffffu, a.v, off);
    r.i = __shfl_xor_sync(0xffffffffu, a.i, off);
    return r;
  }
  // no element compared below (above) the identity: the first one is as good as any
  static __device__ __forceinline__ Out fin(Acc a) { return a.i == 0x7fffffffffffffffll ? 0 : a.i; }
  // Two-pass form for a batch of values a thread visits in index order: one
  // min (max) instruction per value, and only when the batch beats the
  // running value (rare after the first batches) a scan for the first value
  // equal to the batch extreme.
  static constexpr bool kTwoPass = true;
  static constexpr bool kAtomicCols = false;
  static __device__ __forceinline__ T pick(T a, T b) {
    if constexpr (std::is_same<T, float>::value) {
      return MIN ? fminf(a, b) : fmaxf(a, b); // NaNs lose, as they do against `<`
    } else if constexpr (std::is_same<T, double>::value) {
      return MIN ? fmin(a, b) : fmax(a, b);
    } else {
      return MIN ? (b < a ? b : a) : (a < b ? b : a);
    }
  }
  static __device__ __forceinline__ bool beats(T x, T running) { return MIN ? (x < running) : (running < x); }
  // A thread visits its elements in increasing index order, so a strict
  // comparison keeps the first occurrence and a 32-bit visit counter is enough;
  // the 64-bit index is rebuilt once at the end.
  struct Fast {
    T v;
    int k;
  };
  static __device__ __forceinline__ Fast fast_identity() {
    return Fast{MIN ? Limits<T>::highest() : Limits<T>::lowest(), -1};
  }
  static __device__ __forceinline__ void fast_acc(Fast &a, T x, int k) {
    if (MIN ? (x < a.v) : (a.v < x)) {
      a.v = x;
      a.k = k;
    }
  }
  // index_of(k): index along the reduced axis of the thread's visit number k
  template <typename F> static __device__ __forceinline__ Acc widen_fn(Fast f, F index_of) {
    return f.k < 0 ? identity() : Acc{f.v, (int64_t)index_of(f.k)};
  }
};

// L2 (cache-global) load of an accumulator another CTA wrote.
template <typename A> __device__ __forceinline__ A load_cg(const A *p) {
  A r;
  if constexpr (sizeof(A) == 4) {
    int raw = __ldcg(reinterpret_cast<const int *>(p));
    r = *reinterpret_cast<A *>(&raw);
  } else if constexpr (sizeof(A) == 8) {
    long long raw = __ldcg(reinterpret_cast<const long long *>(p));
    r = *reinterpret_cast<A *>(&raw);
  } else {
    static_assert(sizeof(A) == 16, "accumulator size");
    int4 raw = __ldcg(reinterpret_cast<const int4 *>(p));
    r = *reinterpret_cast<A *>(&raw);
  }
  return r;
}

template <typename R> __device__ __forceinline__ typename R::Acc warp_merge(typename R::Acc a) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1)
    a = R::merge(a, R::shfl(a, off));
  return a;
}

// Block-wide merge; every thread calls it, every thread gets the result.
template <typename R>
__device__ __forceinline__ typename R::Acc block_merge(typename R::Acc a, typename R::Acc *scratch) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  a = warp_merge<R>(a);
  __syncthreads();
  if (lane == 0)
    scratch[warp] = a;
  __syncthreads();
  typename R::Acc r = lane < kWarps ? scratch[lane] : R::identity();
  return warp_merge<R>(r);
}

struct Smem {
  unsigned char *tiles;
  uint64_t *full;
  void *scratch;
  __device__ __forceinline__ explicit Smem(unsigned char *raw)
      : tiles(raw), full(reinterpret_cast<uint64_t *>(raw + kStages * kTileBytes)),
        scratch(raw + kStages * kTileBytes + 64) {}
  __device__ __forceinline__ void init() {
    if (threadIdx.x == 0) {
      for (int s = 0; s < kStages; ++s)
        mbar_init(&full[s], 1);
      mbar_init_fence();
    }
    __syncthreads();
  }
};

// Waits for use number `use` of a stage.  A thread whose wait ran out marks
// itself dead (no more waiting, results are garbage) and flags the status word;
// control flow stays uniform so block barriers still match.
__device__ __forceinline__ void stage_wait(uint64_t *bar, int64_t use, bool &dead, uint32_t *status) {
  if (!dead && !mbar_wait(bar, (uint32_t)(use & 1))) {
    dead = true;
    atomicExch(status, (uint32_t)kStatusWaitTimeout);
  }
}

// After a timeout: give copies still in flight a bounded chance to land before
// the CTA's shared memory is released.
__device__ __forceinline__ void drain_after_timeout(Smem &sm, int64_t issued) {
  if (threadIdx.x == 0)
    for (int64_t i = issued > kStages ? issued - kStages : 0; i < issued; ++i)
      (void)mbar_wait(&sm.full[i % kStages], (uint32_t)((i / kStages) & 1));
}

// ---------------------------------------------------------- full reduction ---
// out[0] = reduce(a[0:n]).  CTA b streams the span [b*span, (b+1)*span) with
// span a multiple of the tile size; partials[G] and one counter live in
// scratch memory.  a is 16-byte aligned; the last n % VEC elements are read
// directly by the merging CTA.  With GuardOut the merging CTA leaves out[0]
// untouched when any CTA's bounded wait ran out (the status word is set), for
// callers whose only failure report is that word.
// With px.world > 1 the elements are one GPU's shard: the merging CTA goes on
// to all-reduce out[0] across the GPUs (peer_exchange.cuh).
template <typename R> struct MergeOf {
  using A = typename R::Acc;
  __device__ __forceinline__ A operator()(A a, A b) const { return R::merge(a, b); }
};

template <typename R, bool GuardOut = false>
__device__ __forceinline__ void reduce_all_body(const typename R::In *__restrict__ a,
                                                typename R::Out *__restrict__ out,
                                                typename R::Acc *partials, uint32_t *counter,
                                                int64_t n, int64_t span, uint32_t *status,
                                                unsigned char *smem_raw,
                                                const peer::Args px = peer::Args{nullptr, 0, 0}) {
  using T = typename R::In;
  using Acc = typename R::Acc;
  constexpr int VEC = 16 / sizeof(T);
  constexpr int64_t TILE = kTileBytes / sizeof(T);
  Smem sm(smem_raw);
  T *tiles = reinterpret_cast<T *>(sm.tiles);
  Acc *scratch = reinterpret_cast<Acc *>(sm.scratch);
  sm.init();

  const int tid = threadIdx.x;
  const int64_t G = gridDim.x, b = blockIdx.x;
  const int64_t nvec = n - n % VEC;
  const int64_t begin = b * span < nvec ? b * span : nvec;
  const int64_t end = (b + 1) * span < nvec ? (b + 1) * span : nvec;
  const int64_t ntiles = (end - begin + TILE - 1) / TILE;

  auto issue = [&](int64_t i) {
    const int s = (int)(i % kStages);
    const int64_t e0 = begin + i * TILE;
    const int64_t ne = end - e0 < TILE ? end - e0 : TILE;
    mbar_expect_tx(&sm.full[s], (uint32_t)(ne * sizeof(T)));
    bulk_load(tiles + (int64_t)s * TILE, a + e0, (uint32_t)(ne * sizeof(T)), &sm.full[s]);
  };
  int64_t issued = 0;
  if (tid == 0)
    for (; issued < kStages && issued < ntiles; ++issued)
      issue(issued);

  Acc acc = R::identity();
  bool dead = false;
  for (int64_t i = 0; i < ntiles; ++i) {
    const int s = (int)(i % kStages);
    stage_wait(&sm.full[s], i / kStages, dead, status);
    const int64_t e0 = begin + i * TILE;
    const int64_t ne = end - e0 < TILE ? end - e0 : TILE;
    const T *tile = tiles + (int64_t)s * TILE;
    for (int64_t v = (int64_t)tid * VEC; v < ne; v += kThreads * VEC) {
      const Vec<T, VEC> x = *reinterpret_cast<const Vec<T, VEC> *>(tile + v);
#pragma unroll
      for (int l = 0; l < VEC; ++l)
        R::acc(acc, x.v[l], e0 + v + l);
    }
    __syncthreads();
    if (tid == 0 && issued < ntiles)
      issue(issued++);
  }
  if (__syncthreads_or(dead))
    drain_after_timeout(sm, issued);

  acc = block_merge<R>(acc, scratch);
  __shared__ bool last;
  if (tid == 0) {
    partials[b] = acc;
    __threadfence();
    last = atomicAdd(counter, 1u) == (uint32_t)(G - 1);
  }
  __syncthreads();
  if (!last)
    return;
  __threadfence();
  Acc m = R::identity();
  for (int64_t g = tid; g < G; g += kThreads)
    m = R::merge(m, load_cg(partials + g));
  if (tid == 0)
    for (int64_t e = nvec; e < n; ++e)
      R::acc(m, a[e], e);
  m = block_merge<R>(m, scratch);
  if (tid == 0) {
    if (!GuardOut || load_cg(status) == (uint32_t)kStatusOk)
      out[0] = R::fin(m);
    *counter = 0;
  }
  if constexpr (std::is_same<typename R::Acc, typename R::Out>::value) {
    if (px.world > 1) {
      __syncthreads();
      peer::allreduce_block<typename R::Out>(out, 1, px.peers, px.rank, px.world, status, MergeOf<R>());
    }
  }
}

// ------------------------------------------------ any layout, any alignment ---
// out[o*inner + i] = reduce_k a[o*so + k*sk + i*si] (element strides).
// mode 0: one warp per output, lanes stride over k (reduced axis contiguous);
// mode 1: one thread per output, consecutive threads on consecutive i.
template <typename R>
__device__ __forceinline__ void reduce_generic_body(const typename R::In *__restrict__ a,
                                                    typename R::Out *__restrict__ out, int64_t outer,
                                                    int64_t K, int64_t inner, int64_t so, int64_t sk,
                                                    int64_t si, int mode) {
  using Acc = typename R::Acc;
  const int64_t nout = outer * inner;
  if (mode == 0) {
    const int lane = threadIdx.x & 31;
    const int64_t w = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (w >= nout)
      return;
    const int64_t o = w / inner, i = w % inner;
    Acc acc = R::identity();
    for (int64_t k = lane; k < K; k += 32)
      R::acc(acc, a[o * so + k * sk + i * si], k);
    acc = warp_merge<R>(acc);
    if (lane == 0)
      out[w] = R::fin(acc);
  } else {
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= nout)
      return;
    const int64_t o = t / inner, i = t % inner;
    Acc acc = R::identity();
    for (int64_t k = 0; k < K; ++k)
      R::acc(acc, a[o * so + k * sk + i * si], k);
    out[t] = R::fin(acc);
  }
}

} // namespace red
} // namespace nmb
