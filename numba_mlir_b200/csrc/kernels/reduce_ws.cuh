// Warp-specialised row and column reductions.
//
// One producer warp streams the matrix through a ring of 16 KB shared-memory
// stages with TMA bulk copies (full/empty mbarrier pair per stage); eight
// consumer warps reduce out of shared memory.  There is no block-wide barrier
// in the steady state: a consumer releases a stage as soon as its 128-bit
// reads have landed in registers, and the producer runs ahead by the depth of
// the ring.
#pragma once

#include "reduce_common.cuh"

namespace nmb {
namespace red {

constexpr int kConsumerWarps = 8;
constexpr int kWsThreads = (kConsumerWarps + 1) * 32;
// Row kernel: four warps, each with a private ring of kRowDepth stages of 8 KB
// that it fills itself (lane 0 issues the bulk copy for tile j + kRowDepth as
// soon as the warp has read tile j out of the stage), so no warp ever waits
// for another one and about 160 KB per SM stay in flight.
constexpr int kRowWarps = 4;
constexpr int kRowThreads = kRowWarps * 32;
constexpr int kRowDepth = 6;
constexpr int kRowTileBytes = 8192;
constexpr int kRowStages = kRowWarps * kRowDepth;
constexpr int kColStages = 6;                          // two 99 KB CTAs per SM
constexpr int kRowSmemBytes = kRowStages * kRowTileBytes + kRowStages * 8;
constexpr int kColSmemBytes = kColStages * kTileBytes + 2 * kColStages * 8;
constexpr int kColGroup = 8; // row blocks merged per first-level ticket

template <int STAGES, int STAGE_BYTES> struct Ring {
  unsigned char *tiles;
  uint64_t *full;
  uint64_t *empty;
  __device__ __forceinline__ explicit Ring(unsigned char *raw)
      : tiles(raw), full(reinterpret_cast<uint64_t *>(raw + STAGES * STAGE_BYTES)),
        empty(full + STAGES) {}
  __device__ __forceinline__ void init(uint32_t consumers_per_stage) {
    if (threadIdx.x == 0) {
      for (int s = 0; s < STAGES; ++s) {
        mbar_init(&full[s], 1);
        mbar_init(&empty[s], consumers_per_stage);
      }
      mbar_init_fence();
    }
    __syncthreads();
  }
  // Producer side: after a timeout give the copies in flight a bounded chance
  // to land before the CTA's shared memory is released.
  __device__ __forceinline__ void drain(int64_t issued) {
    for (int64_t i = issued > STAGES ? issued - STAGES : 0; i < issued; ++i)
      (void)mbar_wait(&full[i % STAGES], (uint32_t)((i / STAGES) & 1));
  }
};

// Reduces `count` consecutive elements at `src` (shared memory, 16-byte
// aligned, count % VEC == 0) across the lanes of one warp.  `base` is the index
// of src[0] along the reduced axis.  Every lane gets the merged result.
template <typename R>
__device__ __forceinline__ typename R::Acc warp_reduce_span(const typename R::In *src, int64_t count,
                                                            int64_t base) {
  using T = typename R::In;
  using Acc = typename R::Acc;
  using Fast = typename R::Fast;
  constexpr int VEC = 16 / sizeof(T);
  const int lane = threadIdx.x & 31;
  Fast f[VEC];
#pragma unroll
  for (int l = 0; l < VEC; ++l)
    f[l] = R::fast_identity();
  const int nvec = (int)(count / VEC);
  int k = 0;
#pragma unroll 4
  for (int vi = lane; vi < nvec; vi += 32, ++k) {
    const Vec<T, VEC> x = *reinterpret_cast<const Vec<T, VEC> *>(src + (int64_t)vi * VEC);
#pragma unroll
    for (int l = 0; l < VEC; ++l)
      R::fast_acc(f[l], x.v[l], k);
  }
  Acc acc = R::identity();
#pragma unroll
  for (int l = 0; l < VEC; ++l)
    acc = R::merge(acc, R::widen(f[l], base + (int64_t)lane * VEC + l, 32 * VEC));
  return warp_merge<R>(acc);
}

// ----------------------------------------------------------- row reduction ---
// out[r] = reduce(a[r, :]) for a C-contiguous (rows, cols) matrix whose base is
// 16-byte aligned and whose row size is a multiple of 16 bytes.
// Grid: G <= rows CTAs of kRowThreads; CTA b owns rows [rows*b/G, rows*(b+1)/G).
// Work is cut into groups: `rt` whole rows in one 8 KB tile when a row fits a
// tile, else one row as `tpr` consecutive tiles.  Group g belongs to warp
// g % 4, which loads and reduces it alone (no cross-warp traffic).
template <typename R>
__device__ __forceinline__ void reduce_rows_ws(const typename R::In *__restrict__ a,
                                               typename R::Out *__restrict__ out, int64_t rows,
                                               int64_t cols, uint32_t *status,
                                               unsigned char *smem_raw) {
  using T = typename R::In;
  using Acc = typename R::Acc;
  constexpr int64_t TILE = kRowTileBytes / sizeof(T);
  constexpr int K = kRowDepth;
  T *tiles = reinterpret_cast<T *>(smem_raw);
  uint64_t *full = reinterpret_cast<uint64_t *>(smem_raw + kRowStages * kRowTileBytes);
  if (threadIdx.x == 0) {
    for (int s = 0; s < kRowStages; ++s)
      mbar_init(&full[s], 1);
    mbar_init_fence();
  }
  __syncthreads();

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t G = gridDim.x, b = blockIdx.x;
  const int64_t r_begin = rows * b / G, r_end = rows * (b + 1) / G;
  const int64_t nrows = r_end - r_begin;
  const int64_t tpr = (cols + TILE - 1) / TILE;                           // tiles per row
  const int64_t rt = tpr == 1 ? (TILE / cols > 0 ? TILE / cols : 1) : 1; // rows per tile
  const int64_t ngroups = tpr == 1 ? (nrows + rt - 1) / rt : nrows;
  // this warp's groups: warp, warp + 4, ...; its tiles are numbered j = 0, 1, ...
  const int64_t my_groups = ngroups > warp ? (ngroups - warp + kRowWarps - 1) / kRowWarps : 0;
  const int64_t my_tiles = my_groups * tpr;
  bool dead = false;

  auto issue = [&](int64_t j) {
    const int64_t g = warp + (j / tpr) * kRowWarps, ch = j % tpr;
    const int s = warp * K + (int)(j % K);
    const T *src;
    uint32_t bytes;
    if (tpr == 1) {
      const int64_t r0 = r_begin + g * rt;
      const int64_t nr = r_end - r0 < rt ? r_end - r0 : rt;
      src = a + r0 * cols;
      bytes = (uint32_t)(nr * cols * sizeof(T));
    } else {
      const int64_t c0 = ch * TILE;
      const int64_t ne = cols - c0 < TILE ? cols - c0 : TILE;
      src = a + (r_begin + g) * cols + c0;
      bytes = (uint32_t)(ne * sizeof(T));
    }
    mbar_expect_tx(&full[s], bytes);
    bulk_load(tiles + (int64_t)s * TILE, src, bytes, &full[s]);
  };

  if (lane == 0)
    for (int64_t j = 0; j < K && j < my_tiles; ++j)
      issue(j);

  Acc racc = R::identity();
  for (int64_t j = 0; j < my_tiles; ++j) {
    const int64_t g = warp + (j / tpr) * kRowWarps, ch = j % tpr;
    const int s = warp * K + (int)(j % K);
    stage_wait(&full[s], j / K, dead, status);
    const T *tile = tiles + (int64_t)s * TILE;
    if (tpr == 1) {
      const int64_t r0 = r_begin + g * rt;
      const int nr = (int)(r_end - r0 < rt ? r_end - r0 : rt);
      for (int jr = 0; jr < nr; ++jr) {
        const Acc acc = warp_reduce_span<R>(tile + (int64_t)jr * cols, cols, 0);
        if (lane == 0)
          out[r0 + jr] = R::fin(acc);
      }
    } else {
      const int64_t c0 = ch * TILE;
      const int64_t ne = cols - c0 < TILE ? cols - c0 : TILE;
      racc = R::merge(racc, warp_reduce_span<R>(tile, ne, c0));
      if (ch == tpr - 1) {
        if (lane == 0)
          out[r_begin + g] = R::fin(racc);
        racc = R::identity();
      }
    }
    __syncwarp(); // every lane has its data in registers: the stage is free
    if (lane == 0 && j + K < my_tiles)
      issue(j + K);
  }
  if (dead && lane == 0) // bounded pause (about 2 ms) for copies that may still be in flight
    for (int t = 0; t < 2000; ++t)
      __nanosleep(1000);
}

// -------------------------------------------------------- column reduction ---
// out[c] = reduce(a[:, c]).  Grid (col_tiles, row_blocks) of kWsThreads: CTA
// (x, y) reduces rows [rows*y/Gy, rows*(y+1)/Gy) of the 256*VEC columns that
// start at x*256*VEC; each stage holds 4 row segments (one bulk copy each).
// partials[y][c], then group_partials[ceil(Gy/8)][c], and the ticket counters
// [x][1 + ceil(Gy/8)] live in scratch memory; counters start at zero and are
// left at zero.
template <typename R>
__device__ __forceinline__ void reduce_cols_ws(const typename R::In *__restrict__ a,
                                               typename R::Out *__restrict__ out,
                                               typename R::Acc *partials, uint32_t *counters,
                                               int64_t rows, int64_t cols, uint32_t *status,
                                               unsigned char *smem_raw) {
  using T = typename R::In;
  using Acc = typename R::Acc;
  using Fast = typename R::Fast;
  constexpr int VEC = 16 / sizeof(T);
  constexpr int COLS = kConsumerWarps * 32 * VEC;
  constexpr int RS = kTileBytes / (COLS * (int)sizeof(T));
  constexpr int64_t TILE = kTileBytes / sizeof(T);
  constexpr int S = kColStages;
  Ring<S, kTileBytes> ring(smem_raw);
  T *tiles = reinterpret_cast<T *>(ring.tiles);
  ring.init(kConsumerWarps);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t c0 = (int64_t)blockIdx.x * COLS;
  const int ncols = (int)(cols - c0 < COLS ? cols - c0 : COLS);
  const int64_t Gy = gridDim.y, by = blockIdx.y;
  const int64_t r_begin = rows * by / Gy, r_end = rows * (by + 1) / Gy;
  const int64_t nsteps = (r_end - r_begin + RS - 1) / RS;
  const bool consumer = warp < kConsumerWarps;
  const bool active = consumer && tid * VEC < ncols;
  bool dead = false;

  Fast f[VEC];
#pragma unroll
  for (int l = 0; l < VEC; ++l)
    f[l] = R::fast_identity();

  if (!consumer) {
    if (lane == 0) {
      const uint32_t row_bytes = (uint32_t)(ncols * sizeof(T));
      for (int64_t i = 0; i < nsteps; ++i) {
        const int s = (int)(i % S);
        const int64_t use = i / S;
        if (use > 0)
          stage_wait(&ring.empty[s], use - 1, dead, status);
        const int64_t r0 = r_begin + i * RS;
        const int nr = (int)(r_end - r0 < RS ? r_end - r0 : RS);
        mbar_expect_tx(&ring.full[s], row_bytes * nr);
        for (int j = 0; j < nr; ++j)
          bulk_load(tiles + (int64_t)s * TILE + (int64_t)j * COLS, a + (r0 + j) * cols + c0,
                    row_bytes, &ring.full[s]);
      }
      if (dead)
        ring.drain(nsteps);
    }
  } else {
    for (int64_t i = 0; i < nsteps; ++i) {
      const int s = (int)(i % S);
      stage_wait(&ring.full[s], i / S, dead, status);
      const int64_t r0 = r_begin + i * RS;
      const int nr = (int)(r_end - r0 < RS ? r_end - r0 : RS);
      Vec<T, VEC> x[RS];
      if (active) {
        const T *tile = tiles + (int64_t)s * TILE + tid * VEC;
#pragma unroll
        for (int j = 0; j < RS; ++j)
          if (j < nr)
            x[j] = *reinterpret_cast<const Vec<T, VEC> *>(tile + (int64_t)j * COLS);
      }
      __syncwarp();
      if (lane == 0)
        mbar_arrive(&ring.empty[s]);
      if (active) {
#pragma unroll
        for (int j = 0; j < RS; ++j)
          if (j < nr)
#pragma unroll
            for (int l = 0; l < VEC; ++l)
              R::fast_acc(f[l], x[j].v[l], (int)(i * RS + j));
      }
    }
  }

  Acc acc[VEC];
#pragma unroll
  for (int l = 0; l < VEC; ++l)
    acc[l] = R::widen(f[l], r_begin, 1);

  if (Gy == 1) {
    if (active)
#pragma unroll
      for (int l = 0; l < VEC; ++l)
        out[c0 + tid * VEC + l] = R::fin(acc[l]);
    return;
  }
  // Two-level merge through scratch memory.  Level 1: the last CTA of each
  // group of kColGroup row blocks merges the group's partials (independent
  // loads, merged in row-block order) into group_partials; level 2: the last
  // of those merges the groups.  counters = [x][1 + ngroups] tickets.
  const int64_t ngroups = (Gy + kColGroup - 1) / kColGroup;
  const int64_t grp = by / kColGroup;
  const int64_t g_begin = grp * kColGroup;
  const int64_t g_size = Gy - g_begin < kColGroup ? Gy - g_begin : kColGroup;
  Acc *group_partials = partials + Gy * cols;
  uint32_t *top = counters + (int64_t)blockIdx.x * (1 + ngroups);
  uint32_t *mine = top + 1 + grp;
  __shared__ bool last;

  if (active)
#pragma unroll
    for (int l = 0; l < VEC; ++l)
      partials[by * cols + c0 + tid * VEC + l] = acc[l];
  __threadfence();
  __syncthreads();
  if (tid == 0)
    last = atomicAdd(mine, 1u) == (uint32_t)(g_size - 1);
  __syncthreads();
  if (!last)
    return;
  __threadfence();
  if (active) {
#pragma unroll
    for (int l = 0; l < VEC; ++l) {
      Acc part[kColGroup];
#pragma unroll
      for (int y = 0; y < kColGroup; ++y)
        if (y < g_size)
          part[y] = load_cg(partials + (g_begin + y) * cols + c0 + tid * VEC + l);
      Acc m = R::identity();
#pragma unroll
      for (int y = 0; y < kColGroup; ++y)
        if (y < g_size)
          m = R::merge(m, part[y]);
      group_partials[grp * cols + c0 + tid * VEC + l] = m;
    }
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    *mine = 0;
    last = atomicAdd(top, 1u) == (uint32_t)(ngroups - 1);
  }
  __syncthreads();
  if (!last)
    return;
  __threadfence();
  if (active) {
#pragma unroll
    for (int l = 0; l < VEC; ++l) {
      Acc m = R::identity();
      for (int64_t g0 = 0; g0 < ngroups; g0 += kColGroup) {
        Acc part[kColGroup];
#pragma unroll
        for (int y = 0; y < kColGroup; ++y)
          if (g0 + y < ngroups)
            part[y] = load_cg(group_partials + (g0 + y) * cols + c0 + tid * VEC + l);
#pragma unroll
        for (int y = 0; y < kColGroup; ++y)
          if (g0 + y < ngroups)
            m = R::merge(m, part[y]);
      }
      out[c0 + tid * VEC + l] = R::fin(m);
    }
  }
  if (tid == 0)
    *top = 0;
}

} // namespace red
} // namespace nmb
