// Row and column reductions over a C-contiguous (rows, cols) matrix.
//
// Both kernels stream the matrix through a 4-stage ring of 16 KB shared-memory
// tiles filled by TMA bulk copies (one elected thread issues, an mbarrier per
// stage signals arrival) and keep three 256-thread CTAs per SM, i.e. about
// 150 KB in flight per SM.  Every CTA walks a contiguous range of rows, so
// DRAM sees long sequential streams.  The tile shapes are chosen so that the
// steady state needs no cross-warp exchange:
//
//   rows, wide (row > 2 KB):  a tile is 8 rows x one 2 KB column chunk (eight
//       bulk copies, one issued by each warp); warp w owns row w of the block
//       and accumulates it over the chunks, then five shuffles finish the row.
//   rows, narrow (row <= 2 KB): a tile is a contiguous run of whole rows; the
//       warps take rows w, w+8, ... of the tile.
//   columns: a tile is a contiguous run of whole rows (or one 16 KB piece of a
//       long row); thread t owns the column vectors t, t+256, ... and keeps
//       their accumulators in registers for the CTA's whole row range; CTAs
//       are combined through partials in scratch memory and two levels of
//       ticket counters, merged in index order.
#pragma once

#include "reduce_common.cuh"

namespace nmb {
namespace red {

constexpr int kChunkBytes = 2048; // per-row piece of a wide-row tile
constexpr int kRowsPerBlock = kWarps;
constexpr int kMaxFanIn = 32;      // upper bound of the merge tree's fan-in (a launch parameter)
constexpr int kColVecs = 4;       // column vectors per thread

// ----------------------------------------------------------- row reduction ---
// out[r] = reduce(a[r, :]); base 16-byte aligned, row size a multiple of 16.
// Grid: G CTAs of 256 threads; CTA b owns row blocks (wide) or tiles (narrow)
// [n*b/G, n*(b+1)/G).
template <typename R>
__device__ __forceinline__ void reduce_rows_ws(const typename R::In *__restrict__ a,
                                               typename R::Out *__restrict__ out, int64_t rows,
                                               int64_t cols, uint32_t *status,
                                               unsigned char *smem_raw) {
  using T = typename R::In;
  using Acc = typename R::Acc;
  using Fast = typename R::Fast;
  constexpr int VEC = 16 / sizeof(T);
  constexpr int64_t TILE = kTileBytes / sizeof(T);
  constexpr int64_t CH = kChunkBytes / sizeof(T);   // elements per chunk
  constexpr int VPC = (int)(CH / (32 * VEC));       // vector visits per lane per chunk
  Smem sm(smem_raw);
  T *tiles = reinterpret_cast<T *>(sm.tiles);
  sm.init();

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t G = gridDim.x, b = blockIdx.x;
  bool dead = false;
  int64_t issued = 0;

  if (cols > CH) {
    // ---- wide rows ----------------------------------------------------------
    const int64_t nblocks = (rows + kRowsPerBlock - 1) / kRowsPerBlock;
    const int64_t blk_begin = nblocks * b / G, blk_end = nblocks * (b + 1) / G;
    const int64_t cpr = (cols + CH - 1) / CH; // chunks per row
    const int64_t ntiles = (blk_end - blk_begin) * cpr;

    // Lane 0 of warp w fetches row w's chunk of the tile (a bulk copy costs the
    // issuing thread about 0.1 us, so one thread issuing all eight would hold
    // the CTA back); thread 0 posts the byte count of the whole tile.
    // (row block, chunk) of the next tile to fetch and of the tile being reduced
    // advance with the tile counters: no 64-bit division in the per-tile path
    int64_t iblk = blk_begin, ich = 0, cblk = blk_begin, cch = 0;
    auto issue = [&](int64_t i) {
      const int s = (int)(i % kStages);
      const int64_t r0 = iblk * kRowsPerBlock, c0 = ich * CH;
      if (++ich == cpr) {
        ich = 0;
        ++iblk;
      }
      const int nr = (int)(rows - r0 < kRowsPerBlock ? rows - r0 : kRowsPerBlock);
      const uint32_t bytes = (uint32_t)((cols - c0 < CH ? cols - c0 : CH) * sizeof(T));
      if (tid == 0)
        mbar_expect_tx(&sm.full[s], bytes * nr);
      if (lane == 0 && warp < nr)
        bulk_load(tiles + (int64_t)s * TILE + (int64_t)warp * CH, a + (r0 + warp) * cols + c0, bytes,
                  &sm.full[s]);
    };
    // every thread runs `issue` (so that the counters stay in step); the copies
    // themselves are made by lane 0 of each warp
    for (; issued < kStages && issued < ntiles; ++issued)
      issue(issued);

    Fast f[VEC];
#pragma unroll
    for (int l = 0; l < VEC; ++l)
      f[l] = R::fast_identity();
    int k = 0; // visits of this lane within the current row
    for (int64_t i = 0; i < ntiles; ++i) {
      const int s = (int)(i % kStages);
      stage_wait(&sm.full[s], i / kStages, dead, status);
      const int64_t r = cblk * kRowsPerBlock + warp, ch = cch;
      if (++cch == cpr) {
        cch = 0;
        ++cblk;
      }
      const int64_t c0 = ch * CH;
      const int nvec = (int)((cols - c0 < CH ? cols - c0 : CH) / VEC);
      if (r < rows) {
        const T *src = tiles + (int64_t)s * TILE + (int64_t)warp * CH;
        if constexpr (R::kTwoPass) {
          // index-carrying reducers: extreme of the batch first, position only
          // if the batch wins (visits past the row's end hold the identity)
          Vec<T, VEC> x[VPC];
          int nvis = 0;
#pragma unroll
          for (int v = 0; v < VPC; ++v) {
            const int vi = lane + 32 * v;
            if (vi < nvec) {
              x[v] = *reinterpret_cast<const Vec<T, VEC> *>(src + vi * VEC);
              ++nvis;
            } else {
#pragma unroll
              for (int l = 0; l < VEC; ++l)
                x[v].v[l] = R::fast_identity().v;
            }
          }
#pragma unroll
          for (int l = 0; l < VEC; ++l) {
            T m = x[0].v[l];
#pragma unroll
            for (int v = 1; v < VPC; ++v)
              m = R::pick(m, x[v].v[l]);
            if (R::beats(m, f[l].v)) {
              int first = VPC - 1;
#pragma unroll
              for (int v = VPC - 2; v >= 0; --v)
                first = (x[v].v[l] == m) ? v : first;
              f[l].v = m;
              f[l].k = k + first;
            }
          }
          k += nvis;
        } else {
#pragma unroll
          for (int v = 0; v < VPC; ++v) {
            const int vi = lane + 32 * v;
            if (vi < nvec) {
              const Vec<T, VEC> x = *reinterpret_cast<const Vec<T, VEC> *>(src + vi * VEC);
#pragma unroll
              for (int l = 0; l < VEC; ++l)
                R::fast_acc(f[l], x.v[l], k);
              ++k;
            }
          }
        }
        if (ch == cpr - 1) {
          Acc acc = R::identity();
#pragma unroll
          for (int l = 0; l < VEC; ++l)
            acc = R::merge(acc, R::widen_fn(f[l], [&](int kk) {
              // visit kk of this lane: chunk kk / VPC, vector lane + 32 * (kk % VPC)
              return (int64_t)(kk / VPC) * CH + ((int64_t)lane + 32 * (kk % VPC)) * VEC + l;
            }));
          acc = warp_merge<R>(acc);
          if (lane == 0)
            out[r] = R::fin(acc);
#pragma unroll
          for (int l = 0; l < VEC; ++l)
            f[l] = R::fast_identity();
          k = 0;
        }
      }
      __syncthreads(); // the whole CTA is done with stage s
      if (issued < ntiles)
        issue(issued++);
    }
  } else {
    // ---- narrow rows ----------------------------------------------------------
    const int64_t rt = TILE / cols; // rows per tile (>= 8)
    const int64_t ntiles_all = (rows + rt - 1) / rt;
    const int64_t t_begin = ntiles_all * b / G, t_end = ntiles_all * (b + 1) / G;
    const int64_t ntiles = t_end - t_begin;

    auto issue = [&](int64_t i) {
      const int s = (int)(i % kStages);
      const int64_t r0 = (t_begin + i) * rt;
      const int64_t nr = rows - r0 < rt ? rows - r0 : rt;
      const uint32_t bytes = (uint32_t)(nr * cols * sizeof(T));
      mbar_expect_tx(&sm.full[s], bytes);
      bulk_load(tiles + (int64_t)s * TILE, a + r0 * cols, bytes, &sm.full[s]);
    };
    if (tid == 0)
      for (; issued < kStages && issued < ntiles; ++issued)
        issue(issued);

    const int nvec = (int)(cols / VEC);
    for (int64_t i = 0; i < ntiles; ++i) {
      const int s = (int)(i % kStages);
      stage_wait(&sm.full[s], i / kStages, dead, status);
      const int64_t r0 = (t_begin + i) * rt;
      const int nr = (int)(rows - r0 < rt ? rows - r0 : rt);
      const T *tile = tiles + (int64_t)s * TILE;
      for (int j = warp; j < nr; j += kWarps) {
        Fast f[VEC];
#pragma unroll
        for (int l = 0; l < VEC; ++l)
          f[l] = R::fast_identity();
        int k = 0;
        for (int vi = lane; vi < nvec; vi += 32, ++k) {
          const Vec<T, VEC> x = *reinterpret_cast<const Vec<T, VEC> *>(tile + (int64_t)j * cols + vi * VEC);
#pragma unroll
          for (int l = 0; l < VEC; ++l)
            R::fast_acc(f[l], x.v[l], k);
        }
        Acc acc = R::identity();
#pragma unroll
        for (int l = 0; l < VEC; ++l)
          acc = R::merge(acc, R::widen_fn(f[l], [&](int kk) {
            return ((int64_t)lane + 32 * (int64_t)kk) * VEC + l;
          }));
        acc = warp_merge<R>(acc);
        if (lane == 0)
          out[r0 + j] = R::fin(acc);
      }
      __syncthreads();
      if (tid == 0 && issued < ntiles)
        issue(issued++);
    }
  }
  if (__syncthreads_or(dead))
    drain_after_timeout(sm, issued);
}

// ------------------------------------------ exchange between the GPUs' shards ---
// The last word of the 64 KB counter region every queue's scratch starts with.
constexpr int kExchangeTicket = 16383;

// Called (by every thread) of a CTA that has completed one of the grid's
// gridDim.x column tiles of `out`, columns [c0, c0 + ncols).  With an exchange
// pending, the CTA all-reduces its tile across the GPUs (every tile has its
// own range of the mailbox payload, so the tiles' exchanges run side by
// side); the CTA that completes the grid's last tile closes the call.
template <typename R>
__device__ __forceinline__ void tile_done(typename R::Out *out, int64_t c0, int64_t ncols, uint32_t *grid_ticket,
                                          const peer::Args px, uint32_t *status) {
  if constexpr (std::is_same<typename R::Acc, typename R::Out>::value) {
    if (px.world <= 1)
      return;
    using Out = typename R::Out;
    __shared__ peer::Call call;
    __shared__ bool last_tile;
    __threadfence();
    const unsigned long long off = (unsigned long long)c0 * sizeof(Out);
    if (!peer::args_ok(px.rank, px.world, off + (unsigned long long)ncols * sizeof(Out))) {
      if (threadIdx.x == 0)
        atomicExch(status, (uint32_t)kStatusWaitTimeout);
      return;
    }
    peer::begin(call, px.peers, px.rank, px.world);
    peer::push(call, px.rank, px.world, out + c0, ncols, off);
    peer::pull(call, px.rank, px.world, out + c0, ncols, off, MergeOf<R>(), status);
    __syncthreads();
    if (threadIdx.x == 0) {
      last_tile = atomicAdd(grid_ticket, 1u) == gridDim.x - 1;
      if (last_tile) {
        *grid_ticket = 0;
        peer::end_call(call, px.rank);
      }
    }
  }
}

// -------------------------------------------------------- column reduction ---
// out[c] = reduce(a[:, c]).  Grid (col_tiles, row_blocks) of 256 threads: CTA
// (x, y) reduces rows [rows*y/Gy, rows*(y+1)/Gy) of the columns
// [x*ct, min(cols, (x+1)*ct)); ct (a launch parameter, a multiple of 16 bytes
// and at most 16 KB) is the column-slab width.  A stage holds 16 KB / slab
// size row segments, one bulk copy each (a single copy when the slab spans
// whole rows).  Narrow slabs keep the per-CTA partial rows short, so the merge
// tree below costs one memory round trip per level.
// Scratch: the level buffers of the merge tree (partials[Gy][cols], then
// [ceil(Gy/8)][cols], ... down to 2..8 rows) and the ticket counters, which
// start at zero and are left at zero.
// With px.world > 1 the rows are one GPU's shard: the CTA that finishes a
// column tile exchanges the tile's results with the other GPUs'
// (peer_exchange.cuh), so the reduction over the sharded axis is this one
// launch; one more ticket (the last word of the counter region) tells the last
// of them to close the call.
template <typename R>
__device__ __forceinline__ void reduce_cols_ws(const typename R::In *__restrict__ a,
                                               typename R::Out *__restrict__ out,
                                               typename R::Acc *partials, uint32_t *counters,
                                               int64_t rows, int64_t cols, int64_t ct, int64_t fanin,
                                               uint32_t *status, unsigned char *smem_raw,
                                               const peer::Args px = peer::Args{nullptr, 0, 0}) {
  using T = typename R::In;
  using Acc = typename R::Acc;
  using Fast = typename R::Fast;
  constexpr int VEC = 16 / sizeof(T);
  constexpr int64_t TILE = kTileBytes / sizeof(T);
  Smem sm(smem_raw);
  T *tiles = reinterpret_cast<T *>(sm.tiles);
  sm.init();

  const int tid = threadIdx.x;
  const int64_t CT = ct;
  const int64_t c0 = (int64_t)blockIdx.x * CT;
  const int ncols = (int)(cols - c0 < CT ? cols - c0 : CT);     // this CTA's columns
  const int64_t rs = TILE / CT;                                 // rows per stage
  const bool contiguous = CT == cols;
  const int64_t Gy = gridDim.y, by = blockIdx.y;
  const int64_t r_begin = rows * by / Gy, r_end = rows * (by + 1) / Gy;
  const int64_t nsteps = (r_end - r_begin + rs - 1) / rs;
  const int nvec = ncols / VEC;

  // Scratch counters of this column tile: one word per group of every level of
  // the merge tree (the host sizes the region with the same loop).
  int64_t tickets_per_tile = 0;
  const int64_t F = fanin < 2 ? 2 : (fanin > kMaxFanIn ? kMaxFanIn : fanin);
  for (int64_t n = Gy; n > 1; n = (n + F - 1) / F)
    tickets_per_tile += (n + F - 1) / F;
  uint32_t *ticket = counters + (int64_t)blockIdx.x * tickets_per_tile;

  // Order-independent reducers (min, max) skip the tree: the first row block
  // stores the identity into `out` before it starts streaming and raises the top
  // bit of the tile's first counter; every row block ends with one atomic per
  // column, and the last one to arrive clears the counter again.
  constexpr uint32_t kOutReady = 0x80000000u;
  if constexpr (R::kAtomicCols) {
    if (Gy > 1 && by == 0) {
      for (int e = tid; e < ncols; e += kThreads)
        out[c0 + e] = R::fin(R::identity());
      __threadfence();
      __syncthreads();
      if (tid == 0)
        atomicOr(ticket, kOutReady);
    }
  }

  auto issue = [&](int64_t i) {
    const int s = (int)(i % kStages);
    const int64_t r0 = r_begin + i * rs;
    const int nr = (int)(r_end - r0 < rs ? r_end - r0 : rs);
    const uint32_t row_bytes = (uint32_t)(ncols * sizeof(T));
    // Called by lane 0 of every warp: thread 0 posts the stage's byte count,
    // the row segments are fetched by different warps (a bulk copy costs the
    // issuing thread about 0.1 us).
    if (tid == 0)
      mbar_expect_tx(&sm.full[s], row_bytes * nr);
    if (contiguous) {
      if (tid == 0)
        bulk_load(tiles + (int64_t)s * TILE, a + r0 * cols, row_bytes * nr, &sm.full[s]);
    } else {
      for (int j = tid >> 5; j < nr; j += kWarps)
        bulk_load(tiles + (int64_t)s * TILE + (int64_t)j * ncols, a + (r0 + j) * cols + c0, row_bytes,
                  &sm.full[s]);
    }
  };
  int64_t issued = 0;
  if ((tid & 31) == 0)
    for (; issued < kStages && issued < nsteps; ++issued)
      issue(issued);
  issued = nsteps < kStages ? nsteps : kStages; // the same count in every thread

  Fast f[kColVecs][VEC];
#pragma unroll
  for (int m = 0; m < kColVecs; ++m)
#pragma unroll
    for (int l = 0; l < VEC; ++l)
      f[m][l] = R::fast_identity();

  bool dead = false;
  for (int64_t i = 0; i < nsteps; ++i) {
    const int s = (int)(i % kStages);
    stage_wait(&sm.full[s], i / kStages, dead, status);
    const int64_t r0 = r_begin + i * rs;
    const int nr = (int)(r_end - r0 < rs ? r_end - r0 : rs);
    const T *tile = tiles + (int64_t)s * TILE;
    if (nvec <= kThreads) {
      // slabs of up to 256 column vectors (the usual 4 KB slab): one vector per
      // thread and row, nothing else in the loop
      if (tid < nvec) {
        const T *src = tile + tid * VEC;
        int k = (int)(r0 - r_begin); // row number within this CTA's range
#pragma unroll 4
        for (int j = 0; j < nr; ++j, src += ncols, ++k) {
          const Vec<T, VEC> x = *reinterpret_cast<const Vec<T, VEC> *>(src);
#pragma unroll
          for (int l = 0; l < VEC; ++l)
            R::fast_acc(f[0][l], x.v[l], k);
        }
      }
    } else {
      for (int j = 0; j < nr; ++j) {
        const int k = (int)(r0 - r_begin) + j;
#pragma unroll
        for (int m = 0; m < kColVecs; ++m) {
          const int cv = tid + kThreads * m;
          if (cv < nvec) {
            const Vec<T, VEC> x =
                *reinterpret_cast<const Vec<T, VEC> *>(tile + (int64_t)j * ncols + cv * VEC);
#pragma unroll
            for (int l = 0; l < VEC; ++l)
              R::fast_acc(f[m][l], x.v[l], k);
          }
        }
      }
    }
    __syncthreads();
    if (issued < nsteps) {
      if ((tid & 31) == 0)
        issue(issued);
      ++issued;
    }
  }
  if (__syncthreads_or(dead))
    drain_after_timeout(sm, issued);

  auto widen = [&](int m, int l) {
    return R::widen_fn(f[m][l], [&](int kk) { return r_begin + (int64_t)kk; });
  };

  if (Gy == 1) {
#pragma unroll
    for (int m = 0; m < kColVecs; ++m) {
      const int cv = tid + kThreads * m;
      if (cv < nvec)
#pragma unroll
        for (int l = 0; l < VEC; ++l)
          out[c0 + cv * VEC + l] = R::fin(widen(m, l));
    }
    tile_done<R>(out, c0, ncols, counters + kExchangeTicket, px, status);
    return;
  }

  if constexpr (R::kAtomicCols) {
    __shared__ bool out_ready;
    if (tid == 0) {
      // bounded: the first row block is resident from the start of the grid
      bool ok = false;
      for (int spin = 0; spin < (1 << 22) && !ok; ++spin) {
        uint32_t w;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(w) : "l"(ticket) : "memory");
        ok = (w & kOutReady) != 0;
        if (!ok)
          __nanosleep(64);
      }
      if (!ok)
        atomicExch(status, (uint32_t)kStatusWaitTimeout);
      out_ready = ok;
    }
    __syncthreads();
    if (out_ready) {
#pragma unroll
      for (int m = 0; m < kColVecs; ++m) {
        const int cv = tid + kThreads * m;
        if (cv < nvec)
#pragma unroll
          for (int l = 0; l < VEC; ++l)
            R::atomic_merge(out + c0 + cv * VEC + l, widen(m, l));
      }
    }
    __threadfence();
    __syncthreads();
    __shared__ bool last_block;
    if (tid == 0) {
      const uint32_t arrived = atomicAdd(ticket, 1u) & ~kOutReady;
      last_block = arrived == (uint32_t)(Gy - 1);
      if (last_block)
        atomicExch(ticket, 0u); // everyone has read the flag and added its ticket
    }
    if (px.world > 1) {
      __syncthreads();
      if (last_block)
        tile_done<R>(out, c0, ncols, counters + kExchangeTicket, px, status);
    }
    return;
  }

  // Merge tree through scratch memory, fan-in `fanin` per level (chosen by the
  // host, which sizes the level buffers and the tickets with it): the CTA that
  // draws the last ticket of a group merges the group's rows (independent
  // loads, merged in row order, so the result does not depend on scheduling)
  // into one row of the next level and moves up; the last CTA of the top
  // level writes `out`.  Level buffers follow one another in `partials`
  // ([Gy][cols], [ceil(Gy/fanin)][cols], ...); counters hold, per column tile, the
  // tickets of all groups of all levels, start at zero and are left at zero.
  Acc *level = partials;
  int64_t n = Gy, idx = by;
  __shared__ bool last;

#pragma unroll
  for (int m = 0; m < kColVecs; ++m) {
    const int cv = tid + kThreads * m;
    if (cv < nvec)
#pragma unroll
      for (int l = 0; l < VEC; ++l)
        level[idx * cols + c0 + cv * VEC + l] = widen(m, l);
  }
  while (true) {
    const int64_t ngroups = (n + F - 1) / F;
    const int64_t grp = idx / F, g_begin = grp * F;
    const int g_size = (int)(n - g_begin < F ? n - g_begin : F);
    __threadfence();
    __syncthreads();
    if (tid == 0)
      last = atomicAdd(ticket + grp, 1u) == (uint32_t)(g_size - 1);
    __syncthreads();
    if (!last)
      return;
    __threadfence();
    if (tid == 0)
      ticket[grp] = 0;
    Acc *next = level + n * cols;
    const bool top = ngroups == 1;
    // kMergeBatch elements x kRowBatch rows of independent loads are issued
    // before the first merge, so a level costs a few memory round trips; the
    // batch sizes keep the loaded values in registers.
    constexpr int kMergeBatch = sizeof(Acc) > 8 ? 1 : 2;
    constexpr int kRowBatch = 8;
    for (int e0 = tid; e0 < ncols; e0 += kThreads * kMergeBatch) {
      Acc m[kMergeBatch];
#pragma unroll
      for (int u = 0; u < kMergeBatch; ++u)
        m[u] = R::identity();
#pragma unroll 1
      for (int y0 = 0; y0 < g_size; y0 += kRowBatch) {
        Acc part[kMergeBatch][kRowBatch];
#pragma unroll
        for (int u = 0; u < kMergeBatch; ++u) {
          const int e = e0 + u * kThreads;
#pragma unroll
          for (int y = 0; y < kRowBatch; ++y)
            if (e < ncols && y0 + y < g_size)
              part[u][y] = load_cg(level + (g_begin + y0 + y) * cols + c0 + e);
        }
#pragma unroll
        for (int u = 0; u < kMergeBatch; ++u)
#pragma unroll
          for (int y = 0; y < kRowBatch; ++y)
            if (y0 + y < g_size)
              m[u] = R::merge(m[u], part[u][y]); // row order: the result does not depend on scheduling
      }
#pragma unroll
      for (int u = 0; u < kMergeBatch; ++u) {
        const int e = e0 + u * kThreads;
        if (e < ncols) {
          if (top)
            out[c0 + e] = R::fin(m[u]);
          else
            next[grp * cols + c0 + e] = m[u];
        }
      }
    }
    if (top) {
      tile_done<R>(out, c0, ncols, counters + kExchangeTicket, px, status);
      return;
    }
    ticket += ngroups;
    level = next;
    idx = grp;
    n = ngroups;
  }
}

} // namespace red
} // namespace nmb
