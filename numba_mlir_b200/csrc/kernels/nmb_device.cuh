// Device-side support library for sm_100a.
//
// Included by the hand-written kernels linked into the runtime and handed,
// under the name "nmb_device.cuh", to every NVRTC compilation of generated
// code (fused ufunc chains and @kernel bodies).  It must therefore compile
// without any system header.
#pragma once

#ifdef __CUDACC_RTC__
typedef signed char int8_t;
typedef unsigned char uint8_t;
typedef short int16_t;
typedef unsigned short uint16_t;
typedef int int32_t;
typedef unsigned int uint32_t;
typedef long long int64_t;
typedef unsigned long long uint64_t;
#else
#include <cstdint>
#endif

namespace nmb {

// ---------------------------------------------------------------- vectors ---
// N consecutive elements moved with one (or two, for 8-byte types) 128-bit
// access.  The alignment makes the compiler emit ld/st.global.v4.
template <typename T, int N> struct alignas(sizeof(T) * N <= 16 ? sizeof(T) * N : 16) Vec {
  T v[N];
};

// Streaming (read-once) load: bypass L1 allocation, mark evict-first in L2.
template <typename T, int N>
__device__ __forceinline__ Vec<T, N> load_stream(const T *p) {
  Vec<T, N> r;
  if constexpr (sizeof(T) * N == 16) {
    int4 raw = __ldcs(reinterpret_cast<const int4 *>(p));
    r = *reinterpret_cast<Vec<T, N> *>(&raw);
  } else if constexpr (sizeof(T) * N == 32) {
    int4 raw0 = __ldcs(reinterpret_cast<const int4 *>(p));
    int4 raw1 = __ldcs(reinterpret_cast<const int4 *>(p) + 1);
    *reinterpret_cast<int4 *>(&r.v[0]) = raw0;
    *reinterpret_cast<int4 *>(&r.v[N / 2]) = raw1;
  } else if constexpr (sizeof(T) * N == 8) {
    int2 raw = __ldcs(reinterpret_cast<const int2 *>(p));
    r = *reinterpret_cast<Vec<T, N> *>(&raw);
  } else if constexpr (sizeof(T) * N == 4) {
    int raw = __ldcs(reinterpret_cast<const int *>(p));
    r = *reinterpret_cast<Vec<T, N> *>(&raw);
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i)
      r.v[i] = __ldcs(p + i);
  }
  return r;
}

// Reused (broadcast) load through the read-only path.
template <typename T, int N>
__device__ __forceinline__ Vec<T, N> load_reuse(const T *p) {
  Vec<T, N> r;
  if constexpr (sizeof(T) * N == 16) {
    int4 raw = __ldg(reinterpret_cast<const int4 *>(p));
    r = *reinterpret_cast<Vec<T, N> *>(&raw);
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i)
      r.v[i] = __ldg(p + i);
  }
  return r;
}

template <typename T, int N>
__device__ __forceinline__ void store_stream(T *p, const Vec<T, N> &r) {
  if constexpr (sizeof(T) * N == 16) {
    __stcs(reinterpret_cast<int4 *>(p), *reinterpret_cast<const int4 *>(&r));
  } else if constexpr (sizeof(T) * N == 32) {
    __stcs(reinterpret_cast<int4 *>(p), *reinterpret_cast<const int4 *>(&r.v[0]));
    __stcs(reinterpret_cast<int4 *>(p) + 1,
           *reinterpret_cast<const int4 *>(&r.v[N / 2]));
  } else if constexpr (sizeof(T) * N == 8) {
    __stcs(reinterpret_cast<int2 *>(p), *reinterpret_cast<const int2 *>(&r));
  } else if constexpr (sizeof(T) * N == 4) {
    __stcs(reinterpret_cast<int *>(p), *reinterpret_cast<const int *>(&r));
  } else if constexpr (sizeof(T) == 1) {
    // no streaming store for 1-byte elements (bool results of comparisons)
#pragma unroll
    for (int i = 0; i < N; ++i)
      p[i] = r.v[i];
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i)
      __stcs(p + i, r.v[i]);
  }
}

// i % m for a broadcast operand of m elements: a mask when m is a power of
// two, a 32-bit remainder when both fit, the 64-bit remainder otherwise (the
// branches are uniform over the grid).
__device__ __forceinline__ int64_t wrap_index(int64_t i, int64_t m) {
  if ((m & (m - 1)) == 0)
    return i & (m - 1);
  if (((uint64_t)i | (uint64_t)m) >> 32 == 0)
    return (int64_t)((uint32_t)i % (uint32_t)m);
  return i % m;
}

// ------------------------------------------------- fused elementwise loop ---
// A Chain describes one fused ufunc chain over a flat, C-contiguous output
// index space of n elements:
//
//   struct Chain {
//     struct In  { ... };                     // registers for one vector step
//     struct Out { ... };
//     template <int V> __device__ void load(int64_t i, In &) const;
//     template <int V> __device__ void compute(const In &, Out &) const;
//     template <int V> __device__ void store(int64_t i, const Out &) const;
//   };
//
// V is the number of consecutive elements handled per step (4 when every
// pointer is 16-byte aligned and broadcast extents divide by 4, else 1).
// Every thread issues all loads of its UNROLL steps before the first use so
// that UNROLL x (#inputs) 128-bit requests are in flight per thread; a block
// covers BLOCK*V*UNROLL consecutive elements, each step fully coalesced.
template <int BLOCK, int V, int UNROLL, typename Chain>
__device__ __forceinline__ void eltwise_tile(const Chain &chain, int64_t n) {
  const int64_t tile = (int64_t)BLOCK * V * UNROLL;
  const int64_t base = (int64_t)blockIdx.x * tile + (int64_t)threadIdx.x * V;
  if (base + tile - (int64_t)threadIdx.x * V <= n) {
    // Full tile: no bounds checks.
    typename Chain::template In<V> in[UNROLL];
    typename Chain::template Out<V> out[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
      chain.template load<V>(base + (int64_t)u * BLOCK * V, in[u]);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
      chain.template compute<V>(in[u], out[u]);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
      chain.template store<V>(base + (int64_t)u * BLOCK * V, out[u]);
  } else {
#pragma unroll 1
    for (int u = 0; u < UNROLL; ++u) {
      const int64_t i = base + (int64_t)u * BLOCK * V;
      if (i + V <= n) {
        typename Chain::template In<V> in;
        typename Chain::template Out<V> out;
        chain.template load<V>(i, in);
        chain.template compute<V>(in, out);
        chain.template store<V>(i, out);
      } else {
        // Ragged end: element by element.
        for (int64_t j = i; j < n && j < i + V; ++j) {
          typename Chain::template In<1> in;
          typename Chain::template Out<1> out;
          chain.template load<1>(j, in);
          chain.template compute<1>(in, out);
          chain.template store<1>(j, out);
        }
      }
    }
  }
}

// Number of blocks eltwise_tile needs for n elements.
__host__ __device__ inline int64_t eltwise_grid(int64_t n, int block, int v, int unroll) {
  const int64_t tile = (int64_t)block * v * unroll;
  return (n + tile - 1) / tile;
}

// --------------------------------------------------------- warp / block ops ---
template <typename T, typename Op>
__device__ __forceinline__ T warp_reduce(T v, Op op) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1)
    v = op(v, __shfl_xor_sync(0xffffffffu, v, off));
  return v;
}

struct OpAdd {
  template <typename T> __device__ __forceinline__ T operator()(T a, T b) const { return a + b; }
};
struct OpMul {
  template <typename T> __device__ __forceinline__ T operator()(T a, T b) const { return a * b; }
};
// min/max as the reference defines them: select(a < b, a, b)
// (numba_mlir/mlir/builtin/funcs.py:140-160).
struct OpMin {
  template <typename T> __device__ __forceinline__ T operator()(T a, T b) const { return b < a ? b : a; }
};
struct OpMax {
  template <typename T> __device__ __forceinline__ T operator()(T a, T b) const { return a < b ? b : a; }
};

// Block-wide reduction through warp shuffles and one shared-memory exchange.
// Every thread of the block must call it; all threads receive the result.
// `scratch` holds 32 elements of T.
template <typename T, typename Op>
__device__ __forceinline__ T block_reduce(T v, Op op, T neutral, T *scratch) {
  const int lane = threadIdx.x & 31;
  const int nthreads = blockDim.x * blockDim.y * blockDim.z;
  const int tid = threadIdx.x + blockDim.x * (threadIdx.y + blockDim.y * threadIdx.z);
  const int warp = tid >> 5;
  const int nwarps = (nthreads + 31) >> 5;
  v = warp_reduce(v, op);
  __syncthreads();
  if ((tid & 31) == 0)
    scratch[warp] = v;
  __syncthreads();
  T r = (tid & 31) < nwarps ? scratch[tid & 31] : neutral;
  (void)lane;
  r = warp_reduce(r, op);
  return r;
}

// Work-group reduction that tolerates groups cut short by the global size and
// groups whose size is not a multiple of the warp size.  `full` (uniform over
// the block) selects the shuffle tree; otherwise every remaining work-item
// parks its value in `vals` and the group's first work-item, which always
// exists, combines the values of the active ones in work-item order.  Work-items
// past the global size have left the kernel: a block barrier waits only for
// the threads that have not exited.
template <typename T, typename Op>
__device__ __forceinline__ T group_reduce(T v, Op op, T neutral, T *scratch, void *vals_raw,
                                          const unsigned char *active, bool full) {
  if (full)
    return block_reduce(v, op, neutral, scratch);
  T *vals = reinterpret_cast<T *>(vals_raw);
  const int nthreads = blockDim.x * blockDim.y * blockDim.z;
  const int tid = threadIdx.x + blockDim.x * (threadIdx.y + blockDim.y * threadIdx.z);
  __syncthreads(); // the previous reduction's result has been read
  vals[tid] = v;
  __syncthreads();
  if (tid == 0) {
    T acc = neutral;
    for (int t = 0; t < nthreads; ++t)
      if (active[t])
        acc = op(acc, vals[t]);
    scratch[0] = acc;
  }
  __syncthreads();
  return scratch[0];
}

// ------------------------------------------- reduce(f(inputs)), one pass ---
// A reduction whose operand is an elementwise chain reads the chain's inputs
// once (what the reference gets by fusing the producer into the reduction's
// loop nest, numba_mlir/mlir/tests/test_gpu.py:2198-2224): the generated Chain
// (load and compute as above, one output field `out0`) yields the operand's
// values in registers and they are combined on the way.  `op(acc, x)` is the
// library's sequential step (OpMin/OpMax: select(x < acc), NaNs never win), A
// the accumulator and result type.  Partials of different blocks meet through
// scratch memory and ticket counters that every kernel leaves at zero; the
// block that draws the last ticket combines them in index order, so a result
// does not depend on scheduling.
template <typename A> __device__ __forceinline__ A load_partial(const A *p) {
  if constexpr (sizeof(A) == 4) {
    const int raw = __ldcg(reinterpret_cast<const int *>(p));
    return *reinterpret_cast<const A *>(&raw);
  } else {
    const long long raw = __ldcg(reinterpret_cast<const long long *>(p));
    return *reinterpret_cast<const A *>(&raw);
  }
}

// One step of UNROLL vectors at flat indices i0 + u * stride (all loads issued
// before the first use), folded into acc[l] (l = position inside the vector;
// SPLIT keeps the V positions apart, for column reductions).
template <int V, int UNROLL, bool SPLIT, typename A, typename Op, typename Chain>
__device__ __forceinline__ void reduce_step(const Chain &chain, int64_t i0, int64_t stride, A *acc, Op op) {
  typename Chain::template In<V> in[UNROLL];
  typename Chain::template Out<V> val[UNROLL];
#pragma unroll
  for (int u = 0; u < UNROLL; ++u)
    chain.template load<V>(i0 + (int64_t)u * stride, in[u]);
#pragma unroll
  for (int u = 0; u < UNROLL; ++u)
    chain.template compute<V>(in[u], val[u]);
#pragma unroll
  for (int u = 0; u < UNROLL; ++u)
#pragma unroll
    for (int l = 0; l < V; ++l)
      acc[SPLIT ? l : 0] = op(acc[SPLIT ? l : 0], (A)val[u].out0.v[l]);
}

// out[r] = reduce_k value[r * cols + k].  A row belongs to one warp (or, with
// BLOCK_ROW, to the whole block: few long rows); rows are taken round robin.
// cols % V == 0.
// Every result goes through chain.post(acc) on its way out: the elementwise
// chain that follows the reduction (np.sqrt(np.sum(...)), a mean's division),
// or the identity.
template <int BLOCK, int V, int UNROLL, bool BLOCK_ROW, typename A, typename O, typename Op, typename Chain>
__device__ __forceinline__ void reduce_rows_fused(const Chain &chain, int64_t rows, int64_t cols, O *out, Op op,
                                                  A identity, A *scratch) {
  constexpr int L = BLOCK_ROW ? BLOCK : 32;
  const int t = BLOCK_ROW ? threadIdx.x : (threadIdx.x & 31);
  const int64_t first = BLOCK_ROW ? blockIdx.x : (int64_t)blockIdx.x * (BLOCK / 32) + (threadIdx.x >> 5);
  const int64_t step = BLOCK_ROW ? gridDim.x : (int64_t)gridDim.x * (BLOCK / 32);
  constexpr int64_t span = (int64_t)L * V * UNROLL;
  for (int64_t r = first; r < rows; r += step) {
    A acc = identity;
    const int64_t base = r * cols;
    int64_t k0 = 0;
    for (; k0 + span <= cols; k0 += span)
      reduce_step<V, UNROLL, false>(chain, base + k0 + (int64_t)t * V, (int64_t)L * V, &acc, op);
    for (int64_t k = k0 + (int64_t)t * V; k < cols; k += (int64_t)L * V)
      reduce_step<V, 1, false>(chain, base + k, 0, &acc, op);
    if (BLOCK_ROW) {
      acc = block_reduce(acc, op, identity, scratch);
      if (threadIdx.x == 0)
        out[r] = chain.post(acc);
    } else {
      acc = warp_reduce(acc, op);
      if (t == 0)
        out[r] = chain.post(acc);
    }
  }
}

template <typename T, int N> __device__ T vec_element(const Vec<T, N> &);
template <typename T> __device__ __forceinline__ T neutral_min(); // defined with the @kernel API below
template <typename T> __device__ __forceinline__ T neutral_max();

// out[r] = position of the smallest (MIN) or largest value[r * cols + k] of row
// r, one warp per row, rows taken round robin; cols % V == 0.  A lane visits
// its elements in increasing column order, so a strict comparison keeps the
// first occurrence; between lanes the lower column wins ties.  NaNs never
// compare true and are passed over, as in the library's argmin kernels; a row
// in which nothing beats the identity gives 0.
template <int BLOCK, int V, int UNROLL, bool MIN, typename Chain>
__device__ __forceinline__ void reduce_rows_arg_fused(const Chain &chain, int64_t rows, int64_t cols,
                                                      int64_t *out) {
  using In = typename Chain::template In<V>;
  using Out = typename Chain::template Out<V>;
  using T = decltype(vec_element(Out().out0));
  constexpr int64_t kNone = 0x7fffffffffffffffll;
  const int lane = threadIdx.x & 31;
  const int64_t first = (int64_t)blockIdx.x * (BLOCK / 32) + (threadIdx.x >> 5);
  const int64_t step = (int64_t)gridDim.x * (BLOCK / 32);
  constexpr int64_t span = (int64_t)32 * V * UNROLL;
  auto beats = [](T x, T v) { return MIN ? x < v : v < x; };
  for (int64_t r = first; r < rows; r += step) {
    const int64_t base = r * cols;
    T bv = MIN ? neutral_min<T>() : neutral_max<T>();
    int64_t bi = kNone;
    int64_t k0 = 0;
    for (; k0 + span <= cols; k0 += span) {
      In in[UNROLL];
      Out val[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u)
        chain.template load<V>(base + k0 + (int64_t)(u * 32 + lane) * V, in[u]);
#pragma unroll
      for (int u = 0; u < UNROLL; ++u)
        chain.template compute<V>(in[u], val[u]);
#pragma unroll
      for (int u = 0; u < UNROLL; ++u)
#pragma unroll
        for (int l = 0; l < V; ++l)
          if (beats(val[u].out0.v[l], bv)) {
            bv = val[u].out0.v[l];
            bi = k0 + (int64_t)(u * 32 + lane) * V + l;
          }
    }
    for (int64_t k = k0 + (int64_t)lane * V; k < cols; k += 32 * V) {
      In in;
      Out val;
      chain.template load<V>(base + k, in);
      chain.template compute<V>(in, val);
#pragma unroll
      for (int l = 0; l < V; ++l)
        if (beats(val.out0.v[l], bv)) {
          bv = val.out0.v[l];
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

// out[0] = reduce_i value[i], i < n.  Blocks take tiles of BLOCK*V*UNROLL
// elements round robin; n % V may be anything (the tail is read one by one).
// Returns true in the one block that wrote the result (uniform over the block).
template <int BLOCK, int V, int UNROLL, typename A, typename O, typename Op, typename Chain>
__device__ __forceinline__ bool reduce_all_fused(const Chain &chain, int64_t n, O *out, A *partials,
                                                 uint32_t *counter, Op op, A identity, A *scratch) {
  constexpr int64_t tile = (int64_t)BLOCK * V * UNROLL;
  A acc = identity;
  for (int64_t t0 = (int64_t)blockIdx.x * tile; t0 < n; t0 += (int64_t)gridDim.x * tile) {
    const int64_t base = t0 + (int64_t)threadIdx.x * V;
    if (t0 + tile <= n) {
      reduce_step<V, UNROLL, false>(chain, base, (int64_t)BLOCK * V, &acc, op);
    } else {
      for (int u = 0; u < UNROLL; ++u) {
        const int64_t i = base + (int64_t)u * BLOCK * V;
        if (i + V <= n)
          reduce_step<V, 1, false>(chain, i, 0, &acc, op);
        else
          for (int64_t j = i; j < n; ++j)
            reduce_step<1, 1, false>(chain, j, 0, &acc, op);
      }
    }
  }
  acc = block_reduce(acc, op, identity, scratch);
  __shared__ bool last;
  if (threadIdx.x == 0) {
    partials[blockIdx.x] = acc;
    __threadfence();
    last = atomicAdd(counter, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!last)
    return false;
  __threadfence();
  A m = identity;
  for (unsigned g = threadIdx.x; g < gridDim.x; g += BLOCK)
    m = op(m, load_partial(partials + g));
  m = block_reduce(m, op, identity, scratch);
  if (threadIdx.x == 0) {
    out[0] = chain.post(m);
    *counter = 0;
  }
  return true;
}

template <int N> struct IntTag {
  static constexpr int value = N;
};

// Merges `count` rows of partials (row stride `cols`) for this thread's V
// columns at `c`, eight rows of independent loads at a time, in row order.
template <int V, typename A, typename Op>
__device__ __forceinline__ void merge_partial_rows(const A *rows, int64_t count, int64_t cols, int64_t c, A *m,
                                                   Op op) {
  constexpr int kRows = 8;
  for (int64_t y0 = 0; y0 < count; y0 += kRows) {
    A part[kRows][V];
#pragma unroll
    for (int k = 0; k < kRows; ++k)
#pragma unroll
      for (int l = 0; l < V; ++l)
        if (y0 + k < count)
          part[k][l] = load_partial(rows + (y0 + k) * cols + c + l);
#pragma unroll
    for (int k = 0; k < kRows; ++k)
#pragma unroll
      for (int l = 0; l < V; ++l)
        if (y0 + k < count)
          m[l] = op(m[l], part[k][l]);
  }
}

// out[c] = reduce_r value[r * cols + c].  A block covers BLOCK * V * CV adjacent
// columns: a thread owns CV groups of V adjacent columns, BLOCK * V apart, so
// every row is read in whole 16-byte-per-lane segments and, when the block's
// columns are all of them, as one contiguous stretch.  blockIdx.y splits the
// rows.  The row blocks of a column tile meet in two steps so that no block
// merges more than a few rows: groups of kColFanIn row blocks merge into one
// row each (the block that draws the group's last ticket does it), and the
// block that completes the last group merges the groups' rows into `out`.
// Scratch: partials[gridDim.y + groups][cols]; counters: 1 + groups tickets per
// column tile, left at zero.  cols % V == 0.
constexpr int kColFanIn = 16;

// `wrote` (optional, shared memory): set to 1 in the block that stored the
// tile's final values into `out`.
template <int BLOCK, int V, int CV, int UNROLL, typename A, typename O, typename Op, typename Chain>
__device__ __forceinline__ void reduce_cols_fused(const Chain &chain, int64_t rows, int64_t cols, O *out,
                                                  A *partials, uint32_t *counters, Op op, A identity,
                                                  int *wrote = nullptr) {
  const int64_t c0 = ((int64_t)blockIdx.x * BLOCK * CV + threadIdx.x) * V; // first group; group j at + j * BLOCK * V
  const int64_t Y = gridDim.y, y = blockIdx.y;
  const int64_t r0 = rows * y / Y, r1 = rows * (y + 1) / Y;
  A acc[CV][V];
#pragma unroll
  for (int j = 0; j < CV; ++j)
#pragma unroll
    for (int l = 0; l < V; ++l)
      acc[j][l] = identity;
  auto rows_step = [&](int64_t r, auto unroll_tag) {
    constexpr int U = decltype(unroll_tag)::value;
    typename Chain::template In<V> in[U][CV];
    typename Chain::template Out<V> val[U][CV];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int j = 0; j < CV; ++j)
        if (c0 + (int64_t)j * BLOCK * V < cols)
          chain.template load<V>((r + u) * cols + c0 + (int64_t)j * BLOCK * V, in[u][j]);
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int j = 0; j < CV; ++j)
        if (c0 + (int64_t)j * BLOCK * V < cols) {
          chain.template compute<V>(in[u][j], val[u][j]);
#pragma unroll
          for (int l = 0; l < V; ++l)
            acc[j][l] = op(acc[j][l], (A)val[u][j].out0.v[l]);
        }
  };
  int64_t r = r0;
  for (; r + UNROLL <= r1; r += UNROLL)
    rows_step(r, IntTag<UNROLL>());
  for (; r < r1; ++r)
    rows_step(r, IntTag<1>());
#pragma unroll
  for (int j = 0; j < CV; ++j)
    if (c0 + (int64_t)j * BLOCK * V < cols)
#pragma unroll
      for (int l = 0; l < V; ++l) {
        if (Y == 1)
          out[c0 + (int64_t)j * BLOCK * V + l] = chain.post(acc[j][l]);
        else
          partials[y * cols + c0 + (int64_t)j * BLOCK * V + l] = acc[j][l];
      }
  if (Y == 1) {
    if (wrote && threadIdx.x == 0)
      *wrote = 1;
    return;
  }
  const int64_t groups = (Y + kColFanIn - 1) / kColFanIn;
  const int64_t g = y / kColFanIn;
  const int64_t gsize = Y - g * kColFanIn < kColFanIn ? Y - g * kColFanIn : kColFanIn;
  uint32_t *tickets = counters + (int64_t)blockIdx.x * (groups + 1);
  A *level2 = partials + Y * cols;
  __shared__ bool last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    last = atomicAdd(tickets + 1 + g, 1u) == (unsigned)(gsize - 1);
    if (last)
      tickets[1 + g] = 0;
  }
  __syncthreads();
  if (!last)
    return;
  __threadfence();
#pragma unroll
  for (int j = 0; j < CV; ++j) {
    const int64_t c = c0 + (int64_t)j * BLOCK * V;
    if (c < cols) {
      A m[V];
#pragma unroll
      for (int l = 0; l < V; ++l)
        m[l] = identity;
      merge_partial_rows<V>(partials + g * kColFanIn * cols, gsize, cols, c, m, op);
#pragma unroll
      for (int l = 0; l < V; ++l) {
        if (groups == 1)
          out[c + l] = chain.post(m[l]);
        else
          level2[g * cols + c + l] = m[l];
      }
    }
  }
  if (groups == 1) {
    if (wrote && threadIdx.x == 0)
      *wrote = 1;
    return;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    last = atomicAdd(tickets, 1u) == (unsigned)(groups - 1);
    if (last)
      tickets[0] = 0;
  }
  __syncthreads();
  if (!last)
    return;
  __threadfence();
#pragma unroll
  for (int j = 0; j < CV; ++j) {
    const int64_t c = c0 + (int64_t)j * BLOCK * V;
    if (c < cols) {
      A m[V];
#pragma unroll
      for (int l = 0; l < V; ++l)
        m[l] = identity;
      merge_partial_rows<V>(level2, groups, cols, c, m, op);
#pragma unroll
      for (int l = 0; l < V; ++l)
        out[c + l] = chain.post(m[l]);
    }
  }
  if (wrote && threadIdx.x == 0)
    *wrote = 1;
}

// ----------------------------------------------------- packed float32 ops ---
// sm_100 adds, subtracts and multiplies two float32 values with one
// instruction (add/sub/mul.rn.f32x2 on a 64-bit register pair).  Each half is
// rounded like the scalar instruction, so results are bit-identical; what is
// saved is an issue slot per pair, which is what bounds long elementwise
// chains.  The generated chains call these for two adjacent elements.
// Callers keep a multiply whose product feeds an addition or subtraction
// scalar: the assembler merges mul.f32x2 into a dependent add/sub.f32x2 (a
// fused multiply-add, one rounding instead of two) although both carry .rn.
// Writing the sum as fma.f32x2 with a multiplier of 1 does not prevent it
// (measured: a*b + c still came out fused), so no packed form of "product
// then sum" is offered outside fastmath.
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(unsigned long long r, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(r));
}
__device__ __forceinline__ void add2(float a0, float a1, float b0, float b1, float &r0, float &r1) {
  unsigned long long r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(pack2(a0, a1)), "l"(pack2(b0, b1)));
  unpack2(r, r0, r1);
}
__device__ __forceinline__ void sub2(float a0, float a1, float b0, float b1, float &r0, float &r1) {
  unsigned long long r;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(pack2(a0, a1)), "l"(pack2(b0, b1)));
  unpack2(r, r0, r1);
}
__device__ __forceinline__ void mul2(float a0, float a1, float b0, float b1, float &r0, float &r1) {
  unsigned long long r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(pack2(a0, a1)), "l"(pack2(b0, b1)));
  unpack2(r, r0, r1);
}

__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b,
                                                   unsigned long long c) {
  unsigned long long r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ unsigned long long splat2(float v) { return pack2(v, v); }

// ------------------------------------------------------------------- math ---
// float32 stays float32 (numba_mlir/mlir/builtin/funcs.py:180-227); the CUDA
// functions below are the IEEE-rounded (sqrt, div) or <= 2 ulp (log, exp)
// library versions, never the -use_fast_math intrinsics; erf is this file's own.
// log in float32.  x = m * 2^e with m in [sqrt(1/2), sqrt(2)), f = m - 1 (exact):
//   log(x) = e * ln2 + f - f^2/2 + f^3 * P(f),  P of degree 7,
// a weighted least-squares fit on Chebyshev nodes reweighted towards the
// minimax error of the result, rounded to float32.  Measured over every
// float32 in twelve binades with the FMA sequence emulated: 0.94 ulp at most
// (0.77 in the binade of 1).  Zero, negative, subnormal, infinite and NaN
// arguments take the library's logf.  The pair form computes two values with
// f32x2 instructions: the same operations in the same order, bit-identical
// to the scalar form.
// Coefficients of P, highest power first; the constant term follows.
constexpr float kLogC7 = -0.07634449750185013f, kLogC6 = 0.12761560082435608f, kLogC5 = -0.13160191476345062f,
                kLogC4 = 0.14201760292053223f, kLogC3 = -0.16623356938362122f, kLogC2 = 0.20001226663589478f,
                kLogC1 = -0.2500081956386566f, kLogC0 = 0.3333333134651184f;
constexpr float kLn2Over2p23 = 0.693147182464599609375f * 1.1920928955078125e-07f; // ln2 (float32) * 2^-23, exact
__device__ __forceinline__ bool log_fast_range(float x) {
  // positive, normal, finite
  return (uint32_t)(__float_as_int(x) - 0x00800000) < 0x7f000000u;
}
__device__ __forceinline__ float f_log(float x) {
  if (!log_fast_range(x))
    return logf(x);
  const int ix = __float_as_int(x);
  const int eb = (ix - 0x3f3504f3) & (int)0xff800000; // e * 2^23
  const float f = __fsub_rn(__int_as_float(ix - eb), 1.0f);
  const float s = __fmul_rn(f, f);
  float p = kLogC7;
  p = fmaf(p, f, kLogC6);
  p = fmaf(p, f, kLogC5);
  p = fmaf(p, f, kLogC4);
  p = fmaf(p, f, kLogC3);
  p = fmaf(p, f, kLogC2);
  p = fmaf(p, f, kLogC1);
  p = fmaf(p, f, kLogC0);
  const float t = fmaf(p, f, -0.5f);
  const float r = fmaf(t, s, f);
  return fmaf((float)eb, kLn2Over2p23, r);
}
__device__ __forceinline__ void log_pair(float x0, float x1, float &r0, float &r1) {
  if (!log_fast_range(x0) || !log_fast_range(x1)) {
    r0 = f_log(x0);
    r1 = f_log(x1);
    return;
  }
  const int i0 = __float_as_int(x0), i1 = __float_as_int(x1);
  const int e0 = (i0 - 0x3f3504f3) & (int)0xff800000, e1 = (i1 - 0x3f3504f3) & (int)0xff800000;
  unsigned long long f, s;
  asm("sub.rn.f32x2 %0, %1, %2;"
      : "=l"(f)
      : "l"(pack2(__int_as_float(i0 - e0), __int_as_float(i1 - e1))), "l"(splat2(1.0f)));
  asm("mul.rn.f32x2 %0, %1, %1;" : "=l"(s) : "l"(f));
  unsigned long long p = splat2(kLogC7);
  p = fma2(p, f, splat2(kLogC6));
  p = fma2(p, f, splat2(kLogC5));
  p = fma2(p, f, splat2(kLogC4));
  p = fma2(p, f, splat2(kLogC3));
  p = fma2(p, f, splat2(kLogC2));
  p = fma2(p, f, splat2(kLogC1));
  p = fma2(p, f, splat2(kLogC0));
  const unsigned long long t = fma2(p, f, splat2(-0.5f));
  const unsigned long long r = fma2(t, s, f);
  unpack2(fma2(pack2((float)e0, (float)e1), splat2(kLn2Over2p23), r), r0, r1);
}
__device__ __forceinline__ float f_exp(float x) { return expf(x); }
#ifdef NMB_FASTMATH
// fastmath=True: the approximate instructions (sqrt.approx and rsqrt.approx:
// 1 ulp; div.full: 2 ulp over the whole range), the counterpart of the fast
// floating-point mode the reference sets on its device code for that flag
// (mlir/tests/test_gpu.py:1900-1934).
__device__ __forceinline__ float f_sqrt(float x) {
  float r;
  asm("sqrt.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float f_rsqrt(float x) {
  float r;
  asm("rsqrt.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
#else
__device__ __forceinline__ float f_sqrt(float x) { return __fsqrt_rn(x); }
__device__ __forceinline__ float f_rsqrt(float x) { return __fdiv_rn(1.0f, __fsqrt_rn(x)); }
#endif
// erf in float32, branch free (both ranges are evaluated and one is selected, so
// a warp whose lanes straddle the ranges pays nothing extra):
//   |x| <  1: erf(x) = x + x * p(x^2), p a degree-6 polynomial for erf(x)/x - 1;
//   |x| >= 1: erf(x) = sign(x) * (1 - 2^-u(t)), t = min(|x|, 4), u a degree-6
//             polynomial for -log2(erfc(t)); the result is within half an ulp of
//             1 from t = 3.92 on, and ex2.approx's error is scaled by
//             erfc(t) <= 0.16, so the fast exponential costs at most half an ulp.
// Coefficients: weighted least-squares fits on Chebyshev nodes, reweighted
// towards the minimax error, rounded to float32.  Measured against float64 erf
// with the float32 FMA sequence emulated: 0.98 ulp for |x| < 1 and 1.01 ulp
// (1.5 with the exponential's 2 ulp) above.  NaN propagates, erf(+-0) = +-0,
// erf(+-inf) = +-1.
__device__ __forceinline__ float f_erf(float x) {
  const float t = fabsf(x);
  const float s = x * x;
  float p = 7.853846909711137e-05f;
  p = fmaf(p, s, -0.0008010189048945904f);
  p = fmaf(p, s, 0.00518832728266716f);
  p = fmaf(p, s, -0.026853810995817184f);
  p = fmaf(p, s, 0.1128358542919159f);
  p = fmaf(p, s, -0.3761262595653534f);
  p = fmaf(p, s, 0.12837916612625122f);
  const float small = fmaf(p, x, x);
  const float tc = t > 4.0f ? 4.0f : t; // keeps NaN
  float u = -0.0002688896202016622f;
  u = fmaf(u, tc, 0.004252584185451269f);
  u = fmaf(u, tc, -0.03150571510195732f);
  u = fmaf(u, tc, 0.14875170588493347f);
  u = fmaf(u, tc, 0.9206482768058777f);
  u = fmaf(u, tc, 1.626046061515808f);
  u = fmaf(u, tc, 0.0004926985129714012f);
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-u));
  const float large = copysignf(1.0f - e, x);
  return t < 1.0f ? small : large;
}
// f_erf for two values: the polynomials run as packed FMAs, the same operations
// in the same order as the scalar form (bit-identical results).
__device__ __forceinline__ void erf_pair(float x0, float x1, float &r0, float &r1) {
  const float t0 = fabsf(x0), t1 = fabsf(x1);
  const unsigned long long x = pack2(x0, x1);
  unsigned long long s;
  asm("mul.rn.f32x2 %0, %1, %1;" : "=l"(s) : "l"(x));
  unsigned long long p = splat2(7.853846909711137e-05f);
  p = fma2(p, s, splat2(-0.0008010189048945904f));
  p = fma2(p, s, splat2(0.00518832728266716f));
  p = fma2(p, s, splat2(-0.026853810995817184f));
  p = fma2(p, s, splat2(0.1128358542919159f));
  p = fma2(p, s, splat2(-0.3761262595653534f));
  p = fma2(p, s, splat2(0.12837916612625122f));
  float small0, small1;
  unpack2(fma2(p, x, x), small0, small1);
  const unsigned long long tc = pack2(t0 > 4.0f ? 4.0f : t0, t1 > 4.0f ? 4.0f : t1); // keeps NaN
  unsigned long long u = splat2(-0.0002688896202016622f);
  u = fma2(u, tc, splat2(0.004252584185451269f));
  u = fma2(u, tc, splat2(-0.03150571510195732f));
  u = fma2(u, tc, splat2(0.14875170588493347f));
  u = fma2(u, tc, splat2(0.9206482768058777f));
  u = fma2(u, tc, splat2(1.626046061515808f));
  u = fma2(u, tc, splat2(0.0004926985129714012f));
  float u0, u1, e0, e1;
  unpack2(u, u0, u1);
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(-u0));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(-u1));
  r0 = t0 < 1.0f ? small0 : copysignf(1.0f - e0, x0);
  r1 = t1 < 1.0f ? small1 : copysignf(1.0f - e1, x1);
}
#ifdef NMB_FASTMATH
__device__ __forceinline__ float f_div(float a, float b) {
  float r;
  asm("div.full.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
#else
__device__ __forceinline__ float f_div(float a, float b) { return __fdiv_rn(a, b); }
#endif
__device__ __forceinline__ double f_log(double x) { return log(x); }
__device__ __forceinline__ double f_exp(double x) { return exp(x); }
__device__ __forceinline__ double f_sqrt(double x) { return __dsqrt_rn(x); }
__device__ __forceinline__ double f_erf(double x) { return erf(x); }
__device__ __forceinline__ double f_div(double a, double b) { return __ddiv_rn(a, b); }


// ------------------------------------------------------------ @kernel API ---
// get_global_id(d) = blockIdx.d * blockDim.d + threadIdx.d, the mapping of
// numba_mlir/mlir_compiler/lib/pipelines/LowerToGpu.cpp:1113-1137; dimension 0
// is x, the fastest-varying one.
__device__ __forceinline__ int64_t k_get_local_id(int64_t d, const int64_t *) {
  return d == 0 ? threadIdx.x : d == 1 ? threadIdx.y : threadIdx.z;
}
__device__ __forceinline__ int64_t k_get_group_id(int64_t d, const int64_t *) {
  return d == 0 ? blockIdx.x : d == 1 ? blockIdx.y : blockIdx.z;
}
__device__ __forceinline__ int64_t k_get_local_size(int64_t d, const int64_t *) {
  return d == 0 ? blockDim.x : d == 1 ? blockDim.y : blockDim.z;
}
__device__ __forceinline__ int64_t k_get_global_id(int64_t d, const int64_t *gs) {
  return k_get_group_id(d, gs) * k_get_local_size(d, gs) + k_get_local_id(d, gs);
}
__device__ __forceinline__ int64_t k_get_global_size(int64_t d, const int64_t *gs) { return gs[d]; }

// atomic.add returns the updated value, like the reference's simulator
// (numba_mlir/mlir/kernel_sim.py:24-35).
__device__ __forceinline__ int32_t atomic_add(int32_t *p, int32_t v) { return atomicAdd(p, v) + v; }
__device__ __forceinline__ uint32_t atomic_add(uint32_t *p, uint32_t v) { return atomicAdd(p, v) + v; }
__device__ __forceinline__ int64_t atomic_add(int64_t *p, int64_t v) {
  return (int64_t)atomicAdd(reinterpret_cast<unsigned long long *>(p), (unsigned long long)v) + v;
}
__device__ __forceinline__ uint64_t atomic_add(uint64_t *p, uint64_t v) {
  return (uint64_t)atomicAdd(reinterpret_cast<unsigned long long *>(p), (unsigned long long)v) + v;
}
__device__ __forceinline__ float atomic_add(float *p, float v) { return atomicAdd(p, v) + v; }
__device__ __forceinline__ double atomic_add(double *p, double v) { return atomicAdd(p, v) + v; }

template <typename T> __device__ __forceinline__ T neutral_add() { return T(0); }
template <typename T> __device__ __forceinline__ T neutral_mul() { return T(1); }
template <typename T> __device__ __forceinline__ T neutral_min();
template <typename T> __device__ __forceinline__ T neutral_max();
template <> __device__ __forceinline__ float neutral_min<float>() { return __int_as_float(0x7f800000); }
template <> __device__ __forceinline__ float neutral_max<float>() { return __int_as_float(0xff800000); }
template <> __device__ __forceinline__ double neutral_min<double>() { return __longlong_as_double(0x7ff0000000000000ll); }
template <> __device__ __forceinline__ double neutral_max<double>() { return __longlong_as_double(0xfff0000000000000ll); }
template <> __device__ __forceinline__ int32_t neutral_min<int32_t>() { return 0x7fffffff; }
template <> __device__ __forceinline__ int32_t neutral_max<int32_t>() { return (int32_t)0x80000000; }
template <> __device__ __forceinline__ int64_t neutral_min<int64_t>() { return 0x7fffffffffffffffll; }
template <> __device__ __forceinline__ int64_t neutral_max<int64_t>() { return (int64_t)0x8000000000000000ll; }

// Python's // and % on integers round toward minus infinity.
template <typename T> __device__ __forceinline__ T py_floordiv(T a, T b) {
  if (b == 0)
    return 0;
  T q = a / b;
  if ((a % b != 0) && ((a < 0) != (b < 0)))
    --q;
  return q;
}
template <typename T> __device__ __forceinline__ T py_mod(T a, T b) {
  if (b == 0)
    return 0;
  T r = a % b;
  if (r != 0 && ((r < 0) != (b < 0)))
    r += b;
  return r;
}
__device__ __forceinline__ float py_mod(float a, float b) {
  float r = fmodf(a, b);
  if (r != 0.f && ((r < 0.f) != (b < 0.f)))
    r += b;
  return r;
}
__device__ __forceinline__ double py_mod(double a, double b) {
  double r = fmod(a, b);
  if (r != 0. && ((r < 0.) != (b < 0.)))
    r += b;
  return r;
}

// floor(a / b) the way NumPy's floor_divide computes it for floats: from the
// remainder, so that the quotient and np.remainder agree.
__device__ __forceinline__ float py_floordiv(float a, float b) {
  if (b == 0.f)
    return a / b;
  float mod = fmodf(a, b);
  float div = (a - mod) / b;
  if (mod != 0.f && ((b < 0.f) != (mod < 0.f)))
    div -= 1.f;
  if (div == 0.f)
    return copysignf(0.f, a / b);
  float fl = floorf(div);
  if (div - fl > 0.5f)
    fl += 1.f;
  return fl;
}
__device__ __forceinline__ double py_floordiv(double a, double b) {
  if (b == 0.)
    return a / b;
  double mod = fmod(a, b);
  double div = (a - mod) / b;
  if (mod != 0. && ((b < 0.) != (mod < 0.)))
    div -= 1.;
  if (div == 0.)
    return copysign(0., a / b);
  double fl = floor(div);
  if (div - fl > 0.5)
    fl += 1.;
  return fl;
}
// Shifts by at least the width give 0 (or the sign), as NumPy defines them.
template <typename T> __device__ __forceinline__ T i_shl(T a, T n) {
  return (n < 0 || n >= (T)(8 * sizeof(T))) ? T(0) : (T)(a << n);
}
template <typename T> __device__ __forceinline__ T i_shr(T a, T n) {
  return (n < 0 || n >= (T)(8 * sizeof(T))) ? (a < 0 ? T(-1) : T(0)) : (T)(a >> n);
}
template <typename T> __device__ __forceinline__ T i_sign(T a) { return (T)((a > 0) - (a < 0)); }
__device__ __forceinline__ float f_sign(float a) { return a != a ? a : (float)((a > 0.f) - (a < 0.f)); }
__device__ __forceinline__ double f_sign(double a) { return a != a ? a : (double)((a > 0.) - (a < 0.)); }

// NumPy's maximum/minimum propagate NaNs.
template <typename T> __device__ __forceinline__ T np_max(T a, T b) { return (a > b || a != a) ? a : b; }
template <typename T> __device__ __forceinline__ T np_min(T a, T b) { return (a < b || a != a) ? a : b; }
template <typename T> __device__ __forceinline__ T i_abs(T a) { return a < 0 ? -a : a; }
template <typename T> __device__ __forceinline__ T i_pow(T base, T e) {
  if (e < 0)
    return base == 1 ? 1 : (base == -1 ? ((e & 1) ? -1 : 1) : 0);
  T r = 1;
  while (e) {
    if (e & 1)
      r *= base;
    base *= base;
    e >>= 1;
  }
  return r;
}

} // namespace nmb
