// Dense contraction on the 5th-generation tensor cores (tcgen05 + TMEM) with a
// fused epilogue: the device GEMM entry of the reference
// (numba_mlir/numba_mlir/math_runtime/sycl/lib/NumpyLinalg.cpp:67-176, a oneMKL
// call there) and the pairwise Euclidean distance built on it
// (D = sqrt(max(|x|^2 + |y|^2 - 2 X.Y^T, 0)); reference kernels:
// numba_mlir/mlir/tests/test_gpu.py:1396-1430,2226-2266).
//
// float32 accuracy on TF32 tensor cores comes from the 3xTF32 split: every
// operand is x = hi + lo with hi = tf32(x), lo = tf32(x - hi), and
// X.Y^T ~= hi.hi + hi.lo + lo.hi accumulated in fp32 in TMEM (the dropped
// lo.lo term is 2^-22 relative).
//
// Three kernels:
//   pack      : (rows, K) operand with arbitrary element strides -> per
//               128-row tile, the hi and lo images in the tcgen05 shared-
//               memory operand layout (K-major, no swizzle: 8-row x 16-byte
//               core matrices), zero padded, plus the fp32 row norms.  A
//               whole tile (hi+lo) is then one contiguous TMA bulk copy.
//   contract  : persistent, warp-specialised: warp 0 streams packed tiles in
//               with TMA bulk copies (A resident per row tile, B in four
//               K-half slots of 32 KB), warp 1 issues tcgen05.mma (24 MMAs of
//               128x128x8 per output tile at K = 64, one elected lane of a
//               converged warp) into one of four TMEM accumulators (4 x 128
//               columns = all of TMEM), warps 2-9 drain TMEM with tcgen05.ld
//               in 32 x 32 pieces, apply the epilogue and hand each piece to
//               one asynchronous TMA tensor store out of a private swizzled
//               staging buffer.  The op is store bound (1 GiB out vs 8 MiB in
//               at 16384^2 x 64); the 3xTF32 MMA work (about 0.8 us per tile)
//               runs under the store stream.
//   finish    : the row/column-term epilogue for K > 64, where the dot
//               products are accumulated over K blocks in gemm mode first.
//
// Every wait on an mbarrier is bounded; on a timeout the kernel flags the
// queue's status word, stops, pauses for copies in flight, frees TMEM, returns.

#include "gpu_common.h"
#include "kernels/bulk_pipe.cuh"

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>

#define GPUX_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

constexpr int kTile = 128;         // output tile is kTile x kTile
constexpr int kMaxK = 64;          // K elements resident per launch
constexpr int kChunkBytes = 2048;  // one K chunk (4 elements) of a 128-row tile: 16 groups x 128 B
constexpr int kThreads = 320;      // producer warp, MMA warp, 8 epilogue warps
constexpr int kEpilogueWarps = 8;
constexpr int kEpilogueWarp0 = 2;
constexpr uint64_t kWaitCycles = 4000000000ull; // about 2 s
constexpr int kStageBytes = 65536;  // one operand tile (hi+lo at K = 64) == one 128x128 fp32 output tile

__host__ __device__ inline int padK(int k) { return (k + 7) / 8 * 8; }
// bytes of one part (hi or lo) of a tile image
__host__ __device__ inline int partBytes(int kpad) { return kpad / 4 * kChunkBytes; }

// ------------------------------------------------------------------ pack ---
__device__ __forceinline__ float to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

// One operand of the prepass: element (r, k) at src[r * ldr + k * ldk].
struct PackOperand {
  const float *src;
  int64_t rows, ldr, ldk;
  unsigned char *packed; // [tiles][hi | lo] tile images
  float *norms;          // [tiles * 128] row norms, or NULL
  int tiles;
};

// Prepass for both operands in one launch, one CTA per 128-row tile: the K
// range [k0, k0 + kcount) of the tile goes through shared memory (global reads
// along the operand's unit stride, image writes as whole lines), comes out as
// the hi and lo TF32 images, and, when the K range is the whole K, the row
// norms |x_r|^2 (float64 accumulation over k in order, rounded once) are
// written as well.
constexpr int kPackPitch = kMaxK + 1; // floats per staged row: conflict-free column reads

extern "C" __global__ void __launch_bounds__(256)
    nmb_contract_pack_f32(const PackOperand a, const PackOperand b, int k0, int kcount, int kpad) {
  __shared__ float buf[kTile * kPackPitch];
  const bool first = (int)blockIdx.x < a.tiles;
  const PackOperand &op = first ? a : b;
  const int64_t tile = first ? blockIdx.x : blockIdx.x - a.tiles;
  const bool k_fastest = op.ldk <= op.ldr;
  const bool vec = op.ldk == 1 && op.ldr % 4 == 0 && k0 % 4 == 0 &&
                   (reinterpret_cast<uintptr_t>(op.src) & 15) == 0;
  if (vec) {
    // rows are contiguous and 16-byte aligned: the whole tile is requested
    // before the first value is used (8 x 16 bytes per thread at K = 64)
    const int c4s = kpad / 4, total = kTile * c4s;
    constexpr int kBatch = kTile * (kMaxK / 4) / 256;
    float4 v[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int e = u * 256 + threadIdx.x;
      const int r = e / c4s, c = e % c4s;
      const int64_t row = tile * kTile + r;
      v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (e < total && row < op.rows) {
        const float *src = op.src + row * op.ldr + k0 + c * 4;
        if (c * 4 + 4 <= kcount) {
          v[u] = __ldg(reinterpret_cast<const float4 *>(src));
        } else {
          float *vp = &v[u].x;
          for (int i = 0; i < 4; ++i)
            if (c * 4 + i < kcount)
              vp[i] = __ldg(src + i);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int e = u * 256 + threadIdx.x;
      if (e < total) {
        float *dst = buf + (e / c4s) * kPackPitch + (e % c4s) * 4;
        dst[0] = v[u].x;
        dst[1] = v[u].y;
        dst[2] = v[u].z;
        dst[3] = v[u].w;
      }
    }
  } else {
    for (int base = 0; base < kTile * kpad; base += 4 * 256) {
      float v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int e = base + u * 256 + threadIdx.x;
        const int r = k_fastest ? e / kpad : e % kTile;
        const int k = k_fastest ? e % kpad : e / kTile;
        const int64_t row = tile * kTile + r;
        v[u] = (e < kTile * kpad && row < op.rows && k < kcount)
                   ? __ldg(op.src + row * op.ldr + (int64_t)(k0 + k) * op.ldk)
                   : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int e = base + u * 256 + threadIdx.x;
        if (e < kTile * kpad)
          buf[(k_fastest ? e / kpad : e % kTile) * kPackPitch + (k_fastest ? e % kpad : e / kTile)] = v[u];
      }
    }
  }
  __syncthreads();
  if (op.norms && threadIdx.x < kTile) {
    double s = 0.;
    for (int k = 0; k < kcount; ++k) {
      const double v = (double)buf[threadIdx.x * kPackPitch + k];
      s += v * v;
    }
    op.norms[tile * kTile + threadIdx.x] = (float)s;
  }
  const int pbytes = partBytes(kpad);
  float *hi = reinterpret_cast<float *>(op.packed + tile * 2 * (int64_t)pbytes);
  float *lo = reinterpret_cast<float *>(op.packed + tile * 2 * (int64_t)pbytes + pbytes);
  const int chunks = kpad / 4;
  // image offset of (r, chunk kc) in floats: kc * 512 + (r / 8) * 32 + (r % 8) * 4 = kc * 512 + r * 4
  for (int e = threadIdx.x; e < kTile * chunks; e += blockDim.x) {
    const int kc = e / kTile, r = e % kTile;
    float4 h, l;
    float *hp = &h.x, *lp = &l.x;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float v = buf[r * kPackPitch + kc * 4 + i];
      hp[i] = to_tf32(v);
      lp[i] = to_tf32(v - hp[i]);
    }
    const int off = kc * (kChunkBytes / 4) + r * 4;
    *reinterpret_cast<float4 *>(hi + off) = h;
    *reinterpret_cast<float4 *>(lo + off) = l;
  }
}

// norms[r] = sum_k src[r, k]^2, accumulated in float64 and rounded once;
// entries up to `padded` are zero filled.
extern "C" __global__ void __launch_bounds__(256)
    nmb_contract_norms_f32(const float *__restrict__ src, int64_t rows, int64_t ldr, int64_t ldk,
                           int K, int64_t padded, float *__restrict__ norms) {
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= padded)
    return;
  double s = 0.;
  if (r < rows)
    for (int k = 0; k < K; ++k) {
      const double v = (double)src[r * ldr + (int64_t)k * ldk];
      s += v * v;
    }
  norms[r] = (float)s;
}

// -------------------------------------------------------------- contract ---
// Bounded mbarrier wait on a clock budget (the hardware poll itself suspends
// for a while, so counting polls alone would bound nothing useful).
__device__ __forceinline__ bool wait_bounded(uint64_t *bar, uint32_t parity) {
  if (nmb::mbar_try_wait(bar, parity))
    return true;
  const long long t0 = clock64();
  uint32_t n = 0;
  while (!nmb::mbar_try_wait(bar, parity))
    if ((++n & 63u) == 0 && (uint64_t)(clock64() - t0) > kWaitCycles)
      return false;
  return true;
}

// K-major, no-swizzle shared-memory operand descriptor: core matrix = 8 rows x
// 16 bytes stored contiguously; SBO = distance between 8-row groups (128 B),
// LBO = distance between the two 16-byte K chunks of one MMA (2048 B).
__device__ __forceinline__ uint64_t smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3fff);            // start address, bits [0,14)
  d |= (uint64_t)((kChunkBytes >> 4) & 0x3fff) << 16;    // leading byte offset, bits [16,30)
  d |= (uint64_t)((128 >> 4) & 0x3fff) << 32;            // stride byte offset, bits [32,46)
  d |= (uint64_t)1 << 46;                                // descriptor version (sm_100)
  return d;                                              // layout type 0: no swizzle
}

// kind::tf32, fp32 accumulate, A and B K-major, M = 128, N = 128.
constexpr uint32_t kInstrDesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(kTile >> 3) << 17) |
                                ((uint32_t)(kTile >> 4) << 24);

__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                         uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
               :
               : "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(kInstrDesc), "r"(accumulate)
               : "memory");
}

__device__ __forceinline__ void mma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   nmb::smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tmem_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp gets lane
// (row) base + i, registers = columns.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float *v) {
  uint32_t *r = reinterpret_cast<uint32_t *>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(pred));
  return pred != 0;
}

// Shared -> global tiled TMA store of one box at element coordinates (x, y);
// x * 4 bytes must be a multiple of 16.
__device__ __forceinline__ void tma_store_box(const CUtensorMap *map, const void *src_smem, int x,
                                              int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   map),
               "r"(nmb::smem_u32(src_smem)), "r"(x), "r"(y)
               : "memory");
}

__device__ __forceinline__ float sqrt_approx(float x) {
  float r;
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

struct ContractParams {
  const unsigned char *packedA; // [tiles_m][hi | lo]
  const unsigned char *packedB; // [tiles_n][hi | lo]
  const float *normA;           // mode 0: the row term (|x_i|^2 for distances), padded to tiles_m * 128
  const float *normB;           // mode 0: the column term (|y_j|^2), padded to tiles_n * 128
  float *out;                   // (M, N), row stride ldo elements
  int64_t M, N, ldo;
  int kpad;
  int mode;                     // 0: func(alpha * acc + normA[i] + normB[j]), 1: gemm (alpha, beta)
  int func;                     // mode 0: 0 = identity, 1 = sqrt(max(., 0))
  float alpha, beta;
  uint32_t *status;
  int tma_out;                  // 1: out_map is valid, results leave through TMA stores
  int vec_out;                  // plain stores: base and row pitch allow 16-byte stores
};

constexpr int kAccBuffers = 4;                  // 4 x 128 fp32 columns: all of TMEM
constexpr int kStagePitch = 128;                // bytes per staged row (32 floats)
constexpr int kSlotChunks = 8;                  // K chunks (of 4 elements) per B slot: half of kMaxK
constexpr int kSlotBytes = 2 * kSlotChunks * kChunkBytes; // hi + lo images of a K half: 32 KB
constexpr int kBSlots = 4;                      // 128 KB of B slots
constexpr uint32_t kPiece = 8192;               // bytes per bulk copy
constexpr int kNormSlots = 5;                   // ring of per-tile B norms (128 floats each)
constexpr int kNormSlotBytes = kTile * 4;
constexpr int kStoreRows = 32;                  // rows per TMA store box: one 32 x 32 piece
constexpr int kStagingBytes = kStoreRows * kStagePitch; // one staged piece per epilogue warp

extern "C" __global__ void __launch_bounds__(kThreads, 1)
    nmb_contract_tf32x3(const ContractParams p, const __grid_constant__ CUtensorMap out_map) {
  extern __shared__ __align__(1024) unsigned char smem[];
  const int pbytes = partBytes(p.kpad);
  const int tile_bytes = 2 * pbytes;
  unsigned char *smA = smem;                   // one A tile, resident per tile row
  unsigned char *smB = smem + kStageBytes;     // kBSlots K-half slots
  unsigned char *smStage = smem + 3 * kStageBytes; // kEpilogueWarps x 2 KB
  unsigned char *smNorm = smStage + kEpilogueWarps * kStagingBytes; // kNormSlots x 512 B
  uint64_t *bars = reinterpret_cast<uint64_t *>(smNorm + kNormSlots * kNormSlotBytes);
  uint64_t *a_full = bars + 0, *a_empty = bars + 1;
  uint64_t *b_full = bars + 2, *b_empty = bars + 6;       // [kBSlots] each
  uint64_t *acc_full = bars + 10, *acc_empty = bars + 14; // [kAccBuffers] each
  uint64_t *norm_empty = bars + 18;                       // [kNormSlots]
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 18 + kNormSlots);
  volatile uint32_t *abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t tiles_m = (p.M + kTile - 1) / kTile, tiles_n = (p.N + kTile - 1) / kTile;
  const int64_t total = tiles_m * tiles_n;
  const int64_t t_begin = total * blockIdx.x / gridDim.x, t_end = total * (blockIdx.x + 1) / gridDim.x;
  // This CTA's tiles are t_begin + n, n in [0, count): tile row i, column j
  // stepped along with n (no 64-bit divisions inside the role loops).
  const uint32_t count = (uint32_t)(t_end - t_begin);
  const int64_t i_first = t_begin / tiles_n, j_first = t_begin % tiles_n;

  if (threadIdx.x == 0) {
    nmb::mbar_init(a_full, 1);
    nmb::mbar_init(a_empty, 1);
    for (int s = 0; s < kBSlots; ++s) {
      nmb::mbar_init(&b_full[s], 1);
      nmb::mbar_init(&b_empty[s], 1);
    }
    for (int s = 0; s < kAccBuffers; ++s) {
      nmb::mbar_init(&acc_full[s], 1);
      nmb::mbar_init(&acc_empty[s], kEpilogueWarps); // one arrival per epilogue warp
    }
    for (int s = 0; s < kNormSlots; ++s)
      nmb::mbar_init(&norm_empty[s], kEpilogueWarps);
    *abort_flag = 0;
    nmb::mbar_init_fence();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     nmb::smem_u32(tmem_slot)),
                 "r"(kAccBuffers * kTile)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tmem_fence_before();
  __syncthreads();
  tmem_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto give_up = [&]() {
    *abort_flag = 1;
    atomicExch(p.status, (uint32_t)nmb::kStatusWaitTimeout);
  };

  // B travels in K halves: a slot holds the hi and lo images of 32 K elements
  // (8 chunks each) of one tile; the MMA warp frees a slot after the 12 MMAs
  // that read it, so a reload starts half a tile earlier than with whole-tile
  // stages and four loads are in flight.
  const int nchunks = p.kpad / 4;
  const int halves = nchunks > kSlotChunks ? 2 : 1;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    // The whole warp runs the loop; the copies of one slot are issued by
    // different lanes at once (issuing them one after another from one thread
    // cost most of a microsecond per tile).
    int64_t cur_i = -1, i = i_first, j = j_first;
    uint32_t a_uses = 0, m = 0;
    for (uint32_t n = 0; n < count; ++n, j = (j + 1 == tiles_n ? 0 : j + 1), i += (j == 0)) {
      if (*abort_flag)
        break;
      bool ok = true;
      if (i != cur_i) {
        if (a_uses > 0)
          ok = wait_bounded(a_empty, (uint32_t)((a_uses - 1) & 1));
        if (!__all_sync(0xffffffffu, ok)) {
          if (lane == 0)
            give_up();
          break;
        }
        if (lane == 0)
          nmb::mbar_expect_tx(a_full, (uint32_t)tile_bytes);
        __syncwarp();
        for (uint32_t off = (uint32_t)lane * kPiece; off < (uint32_t)tile_bytes; off += 32 * kPiece)
          nmb::bulk_load(smA + off, p.packedA + i * (int64_t)tile_bytes + off,
                         (uint32_t)tile_bytes - off < kPiece ? (uint32_t)tile_bytes - off : kPiece, a_full);
        cur_i = i;
        ++a_uses;
      }
      for (int h = 0; h < halves; ++h, ++m) {
        const int slot = (int)(m % kBSlots);
        const uint32_t use = m / kBSlots;
        if (use > 0)
          ok = wait_bounded(&b_empty[slot], (uint32_t)((use - 1) & 1));
        // the tile's B norms travel with its first half, into a ring slot the
        // epilogue frees
        const int r = (int)(n % kNormSlots);
        const uint32_t r_use = n / kNormSlots;
        const bool with_norms = h == 0 && p.mode == 0;
        if (ok && with_norms && r_use > 0)
          ok = wait_bounded(&norm_empty[r], (uint32_t)((r_use - 1) & 1));
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0)
            give_up();
          break;
        }
        const int ch = nchunks - h * kSlotChunks < kSlotChunks ? nchunks - h * kSlotChunks : kSlotChunks;
        const uint32_t part = (uint32_t)ch * kChunkBytes; // bytes of the hi (or lo) part
        if (lane == 0)
          nmb::mbar_expect_tx(&b_full[slot], 2 * part + (with_norms ? kNormSlotBytes : 0));
        __syncwarp();
        const int per = (int)((part + kPiece - 1) / kPiece); // pieces per part: 1 or 2
        if (lane < 2 * per) {
          const int which = lane / per;                      // 0: hi, 1: lo
          const uint32_t off = (uint32_t)(lane % per) * kPiece;
          nmb::bulk_load(smB + slot * kSlotBytes + which * (kSlotBytes / 2) + off,
                         p.packedB + j * (int64_t)tile_bytes + which * pbytes +
                             h * (kSlotBytes / 2) + off,
                         part - off < kPiece ? part - off : kPiece, &b_full[slot]);
        } else if (lane == 4 && with_norms) {
          nmb::bulk_load(smNorm + r * kNormSlotBytes, p.normB + j * kTile, kNormSlotBytes, &b_full[slot]);
        }
      }
      if (!ok)
        break;
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    // The whole warp runs the loop and the waits in lockstep and one elected
    // lane issues: MMAs issued from a divergent single-lane branch went out
    // at half the rate.
    int64_t cur_i = -1, i = i_first, j = j_first;
    uint32_t a_uses = 0, m = 0;
    // Descriptors differ only in the start-address field (units of 16 bytes):
    // a K step is 2 chunks of 2 KB = 256 units, a K half 8 chunks = 1024.
    constexpr uint64_t kStepUnits = (2 * kChunkBytes) >> 4;
    constexpr uint64_t kHalfUnits = (kSlotChunks * kChunkBytes) >> 4;
    const uint64_t a_hi = smem_desc(nmb::smem_u32(smA)), a_lo = smem_desc(nmb::smem_u32(smA) + pbytes);
    for (uint32_t n = 0; n < count; ++n, j = (j + 1 == tiles_n ? 0 : j + 1), i += (j == 0)) {
      if (*abort_flag)
        break;
      const int buf = (int)(n % kAccBuffers);
      const uint32_t buf_use = n / kAccBuffers;
      const bool last_of_row = (n + 1 == count) || (j + 1 == tiles_n);
      bool ok = true;
      if (i != cur_i) {
        ok = wait_bounded(a_full, (uint32_t)(a_uses & 1));
        cur_i = i;
        ++a_uses;
      }
      if (ok && buf_use > 0)
        ok = wait_bounded(&acc_empty[buf], (uint32_t)((buf_use - 1) & 1));
      for (int h = 0; h < halves; ++h, ++m) {
        const int slot = (int)(m % kBSlots);
        ok = ok && wait_bounded(&b_full[slot], (uint32_t)((m / kBSlots) & 1));
        if (!__all_sync(0xffffffffu, ok)) {
          ok = false;
          break;
        }
        tmem_fence_after();
        if (elect_one()) {
          const int ch = nchunks - h * kSlotChunks < kSlotChunks ? nchunks - h * kSlotChunks : kSlotChunks;
          const int ksteps = ch / 2;
          const uint32_t d_tmem = tmem_base + (uint32_t)(buf * kTile);
          const uint32_t b_addr = nmb::smem_u32(smB + slot * kSlotBytes);
          const uint64_t b_hi = smem_desc(b_addr), b_lo = smem_desc(b_addr + kSlotBytes / 2);
          const uint64_t ah = a_hi + h * kHalfUnits, al = a_lo + h * kHalfUnits;
          // hi.hi (the tile's very first MMA overwrites the accumulator), hi.lo, lo.hi
          uint64_t da = ah, db = b_hi;
          mma_tf32(d_tmem, da, db, h == 0 ? 0u : 1u);
#pragma unroll
          for (int ks = 1; ks < ksteps; ++ks)
            mma_tf32(d_tmem, da += kStepUnits, db += kStepUnits, 1);
          da = ah;
          db = b_lo;
#pragma unroll
          for (int ks = 0; ks < ksteps; ++ks, da += kStepUnits, db += kStepUnits)
            mma_tf32(d_tmem, da, db, 1);
          da = al;
          db = b_hi;
#pragma unroll
          for (int ks = 0; ks < ksteps; ++ks, da += kStepUnits, db += kStepUnits)
            mma_tf32(d_tmem, da, db, 1);
          mma_commit(&b_empty[slot]);      // slot reusable once these MMAs have read it
          if (h == halves - 1) {
            mma_commit(&acc_full[buf]);    // accumulator ready for the epilogue
            if (last_of_row)
              mma_commit(a_empty);
          }
        }
        __syncwarp();
      }
      if (!ok) {
        if (lane == 0)
          give_up();
        break;
      }
    }
  } else {
    // ---------------- epilogue: TMEM -> registers -> shared -> HBM ----------------
    // Warp w may read TMEM lanes 32*(w%4)..+31 (32 rows of the tile); the two
    // warps of a lane quarter take 64 columns each, as two 32 x 32 pieces.
    // A piece leaves as one asynchronous TMA tensor store out of the warp's
    // private 4 KB staging buffer (16-byte chunk k of row r at position
    // k ^ (r & 7), the 128-byte swizzle the tensor map undoes: conflict-free
    // writes), so the warp loads and computes its next piece while the store
    // drains; it waits for the buffer only before restaging.  Outputs the
    // tensor map cannot describe take plain stores.
    const int e = warp - kEpilogueWarp0;
    const int q = warp & 3;
    const int half = e >> 2;
    unsigned char *stage = smStage + e * kStagingBytes;
    int64_t xa_row = -1;
    float xa = 0.f;
    int64_t i = i_first, j = j_first;
    for (uint32_t n = 0; n < count; ++n, j = (j + 1 == tiles_n ? 0 : j + 1), i += (j == 0)) {
      const int buf = (int)(n % kAccBuffers);
      const uint32_t buf_use = n / kAccBuffers;
      const int64_t row0 = i * kTile + q * 32; // first row of this warp's pieces
      const int64_t row = row0 + lane;
      if (p.mode == 0 && row != xa_row) {
        xa = p.normA[row];
        xa_row = row;
      }
      if (!wait_bounded(&acc_full[buf], (uint32_t)(buf_use & 1))) {
        give_up();
        break;
      }
      tmem_fence_after();
      // both pieces into registers; the accumulator is free from then on
      float w0[32], w1[32];
      const uint32_t tsrc = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * kTile + half * 64);
      tmem_ld32(tsrc, w0);
      tmem_ld32(tsrc + 32, w1);
      tmem_ld_wait();
      tmem_fence_before();
      __syncwarp();
      if (lane == 0)
        nmb::mbar_arrive(&acc_empty[buf]);
      const int r = (int)(n % kNormSlots);
      auto finish_piece = [&](float(&w)[32], int pc) {
        const int64_t col0 = j * kTile + half * 64 + pc * 32;
        if (p.mode == 0) {
          // |y_j|^2 of the piece's 32 columns: broadcast reads of the ring slot
          const float4 *y = reinterpret_cast<const float4 *>(smNorm + r * kNormSlotBytes) + half * 16 + pc * 8;
          const float al = p.alpha;
          if (p.func == 1) {
#pragma unroll
            for (int e4 = 0; e4 < 8; ++e4) {
              const float4 yv = y[e4];
              w[e4 * 4 + 0] = sqrt_approx(fmaxf(fmaf(al, w[e4 * 4 + 0], xa + yv.x), 0.f));
              w[e4 * 4 + 1] = sqrt_approx(fmaxf(fmaf(al, w[e4 * 4 + 1], xa + yv.y), 0.f));
              w[e4 * 4 + 2] = sqrt_approx(fmaxf(fmaf(al, w[e4 * 4 + 2], xa + yv.z), 0.f));
              w[e4 * 4 + 3] = sqrt_approx(fmaxf(fmaf(al, w[e4 * 4 + 3], xa + yv.w), 0.f));
            }
          } else {
#pragma unroll
            for (int e4 = 0; e4 < 8; ++e4) {
              const float4 yv = y[e4];
              w[e4 * 4 + 0] = fmaf(al, w[e4 * 4 + 0], xa + yv.x);
              w[e4 * 4 + 1] = fmaf(al, w[e4 * 4 + 1], xa + yv.y);
              w[e4 * 4 + 2] = fmaf(al, w[e4 * 4 + 2], xa + yv.z);
              w[e4 * 4 + 3] = fmaf(al, w[e4 * 4 + 3], xa + yv.w);
            }
          }
        } else {
          const float *orow = p.out + row * p.ldo;
#pragma unroll
          for (int k = 0; k < 32; ++k) {
            float v = p.alpha * w[k];
            if (p.beta != 0.f && row < p.M && col0 + k < p.N)
              v = fmaf(p.beta, orow[col0 + k], v);
            w[k] = v;
          }
        }
        if (p.tma_out) {
          if (lane == 0)
            nmb::bulk_wait_read<0>(); // the previous store has read the buffer
          __syncwarp();
#pragma unroll
          for (int k = 0; k < 8; ++k)
            *reinterpret_cast<float4 *>(stage + lane * kStagePitch + ((k ^ (lane & 7)) << 4)) =
                make_float4(w[k * 4], w[k * 4 + 1], w[k * 4 + 2], w[k * 4 + 3]);
          nmb::fence_async_smem();
          __syncwarp();
          if (lane == 0 && row0 < p.M && col0 < p.N) {
            tma_store_box(&out_map, stage, (int)col0, (int)row0);
            nmb::bulk_commit();
          }
        } else {
          // plain stores, through the same staging buffer so that they leave
          // coalesced: eight lanes write the 128 bytes of one row, a warp
          // instruction four rows (for the 16384 x 16384 distance matrix this
          // path took 268 us where the TMA stores take 234 us on the same GPU)
          __syncwarp(); // the previous piece's reads of the buffer are done
#pragma unroll
          for (int k = 0; k < 8; ++k)
            *reinterpret_cast<float4 *>(stage + lane * kStagePitch + ((k ^ (lane & 7)) << 4)) =
                make_float4(w[k * 4], w[k * 4 + 1], w[k * 4 + 2], w[k * 4 + 3]);
          __syncwarp();
          const int c = lane & 7;
          const int64_t col = col0 + c * 4;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const int rr = k * 4 + (lane >> 3);
            const float4 v = *reinterpret_cast<const float4 *>(stage + rr * kStagePitch + ((c ^ (rr & 7)) << 4));
            const int64_t orow_i = row0 + rr;
            if (orow_i < p.M) {
              float *dst = p.out + orow_i * p.ldo + col;
              if (p.vec_out && col + 3 < p.N) {
                __stcs(reinterpret_cast<float4 *>(dst), v);
              } else {
                if (col < p.N)
                  dst[0] = v.x;
                if (col + 1 < p.N)
                  dst[1] = v.y;
                if (col + 2 < p.N)
                  dst[2] = v.z;
                if (col + 3 < p.N)
                  dst[3] = v.w;
              }
            }
          }
        }
      };
      finish_piece(w0, 0);
      finish_piece(w1, 1);
      __syncwarp();
      if (lane == 0)
        nmb::mbar_arrive(&norm_empty[r]);
    }
    if (lane == 0)
      nmb::bulk_wait_all<0>(); // shared memory must outlive the stores reading it
    __syncwarp();
  }

  tmem_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) // bounded pause (about 2 ms) for copies or MMAs in flight
    for (int t = 0; t < 2000; ++t)
      __nanosleep(1000);
  __syncthreads();
  if (warp == 1) {
    tmem_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(kAccBuffers * kTile)
                 : "memory");
  }
}

// out[i, j] = func(alpha * out[i, j] + na[i] + nb[j]) over an (M, N) matrix.
extern "C" __global__ void __launch_bounds__(256)
    nmb_contract_finish_rowcol(float *out, int64_t M, int64_t N, int64_t ldo,
                               const float *__restrict__ na, const float *__restrict__ nb, float alpha,
                               int func) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= M * N)
    return;
  const int64_t i = idx / N, j = idx % N;
  float *o = out + i * ldo + j;
  const float v = fmaf(alpha, *o, na[i] + nb[j]);
  *o = func == 1 ? sqrt_approx(fmaxf(v, 0.f)) : v;
}

// ------------------------------------------------------------ host side ---
struct Operand {
  const float *data; // element (r, k) at data[r * ldr + k * ldk]
  int64_t rows, K, ldr, ldk;
};

int smCount(int device) {
  static int cached[64] = {0};
  if (device < 64 && cached[device])
    return cached[device];
  int n = 148;
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device);
  if (device < 64)
    cached[device] = n;
  return n;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's entry-point lookup (the library
// does not link against the driver); NULL when the driver lacks it.
EncodeTiledFn encodeTiled() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void *f = nullptr;
    cudaDriverEntryPointQueryResult st;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &st) != cudaSuccess ||
        st != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

size_t alignUp(size_t x, size_t a) { return (x + a - 1) / a * a; }

// What mode 0 adds to alpha * A.B^T: a row term and a column term, each either
// absent, the squared norms of the operand's rows (from the packing prepass) or
// a contiguous vector the caller gives, and the final function.
enum { kTermNone = 0, kTermNorms = 1, kTermVector = 2 };
struct RowCol {
  int rowKind = kTermNone, colKind = kTermNone;
  const float *rowv = nullptr, *colv = nullptr;
  int func = 0; // 0: identity, 1: sqrt(max(., 0))
};

// Fills a padded term vector: `n` values from `src` (or zeros), zeros up to `padded`.
bool fillTerm(float *dst, const float *src, int64_t n, int64_t padded, cudaStream_t stream) {
  cudaError_t e = cudaSuccess;
  if (src)
    e = cudaMemcpyAsync(dst, src, (size_t)n * 4, cudaMemcpyDeviceToDevice, stream);
  const int64_t z0 = src ? n : 0;
  if (e == cudaSuccess && padded > z0)
    e = cudaMemsetAsync(dst + z0, 0, (size_t)(padded - z0) * 4, stream);
  if (e != cudaSuccess) {
    nmb::setError("contraction: filling a row/column term failed: %s", cudaGetErrorString(e));
    return false;
  }
  return true;
}

// Runs out = epilogue(A . B^T) with A (M, K), B (N, K) given as Operands.
// mode 0: out = func(alpha * A.B^T + row term + column term) (`rc`);
// mode 1: out = alpha * A.B^T + beta * out.
bool runContraction(void *queue, const Operand &A, const Operand &B, float *out, int64_t ldo, int mode,
                    float alpha, float beta, const RowCol &rc = RowCol()) {
  nmb::QueueView qv;
  if (!nmb::queueView(queue, &qv))
    return false;
  cudaStream_t stream = static_cast<cudaStream_t>(qv.stream);
  const int64_t M = A.rows, N = B.rows, K = A.K;
  if (M == 0 || N == 0)
    return true;
  const int64_t tiles_m = (M + kTile - 1) / kTile, tiles_n = (N + kTile - 1) / kTile;
  const int kblock = (int)(K < kMaxK ? K : kMaxK);
  const int kpad_max = padK(kblock > 0 ? kblock : 1);
  const size_t packA = (size_t)tiles_m * 2 * partBytes(kpad_max);
  const size_t packB = (size_t)tiles_n * 2 * partBytes(kpad_max);
  const size_t normA = alignUp((size_t)tiles_m * kTile * 4, 256);
  const size_t normB = alignUp((size_t)tiles_n * kTile * 4, 256);
  unsigned char *scratch =
      static_cast<unsigned char *>(nmb::scratchGet(queue, packA + packB + normA + normB + 256));
  if (!scratch)
    return false;
  unsigned char *dA = scratch, *dB = scratch + packA;
  float *nA = reinterpret_cast<float *>(scratch + packA + packB);
  float *nB = reinterpret_cast<float *>(scratch + packA + packB + normA);
  uint32_t *status = nmb::statusWord(queue);
  if (!status)
    return false;

  static bool attrSet[64] = {false};
  const int smemBytes = 3 * kStageBytes + kEpilogueWarps * kStagingBytes + kNormSlots * kNormSlotBytes + 256;
  if (qv.device >= 64 || !attrSet[qv.device]) {
    if (cudaFuncSetAttribute(nmb_contract_tf32x3, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             smemBytes) != cudaSuccess) {
      nmb::setError("cudaFuncSetAttribute(nmb_contract_tf32x3) failed: %s",
                    cudaGetErrorString(cudaGetLastError()));
      return false;
    }
    if (qv.device < 64)
      attrSet[qv.device] = true;
  }

  const bool single = K <= kMaxK;
  if (mode == 0) {
    // terms that do not come from the prepass: given vectors and absent terms
    // (zeros), padded to whole tiles; with K in several blocks the norms over
    // the whole K come from their own kernel
    if (rc.rowKind != kTermNorms && !fillTerm(nA, rc.rowKind == kTermVector ? rc.rowv : nullptr, M,
                                              tiles_m * kTile, stream))
      return false;
    if (rc.colKind != kTermNorms && !fillTerm(nB, rc.colKind == kTermVector ? rc.colv : nullptr, N,
                                              tiles_n * kTile, stream))
      return false;
    if (!single && rc.rowKind == kTermNorms) {
      nmb_contract_norms_f32<<<(unsigned)((tiles_m * kTile + 255) / 256), 256, 0, stream>>>(
          A.data, M, A.ldr, A.ldk, (int)K, tiles_m * kTile, nA);
      nmb::noteLaunch();
    }
    if (!single && rc.colKind == kTermNorms) {
      nmb_contract_norms_f32<<<(unsigned)((tiles_n * kTile + 255) / 256), 256, 0, stream>>>(
          B.data, N, B.ldr, B.ldk, (int)K, tiles_n * kTile, nB);
      nmb::noteLaunch();
    }
  }
  // Tensor map of the output for the epilogue's TMA stores: needs a 16-byte
  // aligned base and row pitch and 32-bit coordinates.
  CUtensorMap out_map;
  memset(&out_map, 0, sizeof(out_map));
  bool tma_out = (reinterpret_cast<uintptr_t>(out) & 15) == 0 && ldo % 4 == 0 && ldo >= N &&
                 M < (1ll << 31) && N < (1ll << 31) && ldo < (1ll << 36);
  if (tma_out) {
    EncodeTiledFn enc = encodeTiled();
    const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)ldo * 4};
    const cuuint32_t box[2] = {32, (cuuint32_t)kStoreRows};
    const cuuint32_t estr[2] = {1, 1};
    tma_out = enc && enc(&out_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, out, dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_NONE,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
  }
  const int64_t total = tiles_m * tiles_n;
  const int64_t sms = smCount(qv.device);
  const unsigned grid = (unsigned)(total < sms ? total : sms);
  int64_t k0 = 0;
  bool first = true;
  do {
    const int kcount = (int)(K - k0 < kMaxK ? K - k0 : kMaxK);
    const int kpad = padK(kcount > 0 ? kcount : 1);
    const bool fused_norms = mode == 0 && single;
    const PackOperand pa{A.data, M, A.ldr, A.ldk, dA, fused_norms && rc.rowKind == kTermNorms ? nA : nullptr,
                         (int)tiles_m};
    const PackOperand pb{B.data, N, B.ldr, B.ldk, dB, fused_norms && rc.colKind == kTermNorms ? nB : nullptr,
                         (int)tiles_n};
    nmb_contract_pack_f32<<<(unsigned)(tiles_m + tiles_n), 256, 0, stream>>>(pa, pb, (int)k0, kcount,
                                                                             kpad);
    ContractParams p;
    p.packedA = dA;
    p.packedB = dB;
    p.normA = nA;
    p.normB = nB;
    p.out = out;
    p.M = M;
    p.N = N;
    p.ldo = ldo;
    p.kpad = kpad;
    p.status = status;
    p.tma_out = tma_out ? 1 : 0;
    p.vec_out = (reinterpret_cast<uintptr_t>(out) & 15) == 0 && ldo % 4 == 0 ? 1 : 0;
    p.func = rc.func;
    if (mode == 0 && single) {
      p.mode = 0;
      p.alpha = alpha;
      p.beta = 0.f;
    } else {
      p.mode = 1;
      p.alpha = mode == 0 ? 1.f : alpha;
      p.beta = first ? (mode == 0 ? 0.f : beta) : 1.f;
    }
    nmb_contract_tf32x3<<<grid, kThreads, smemBytes, stream>>>(p, out_map);
    nmb::noteLaunch();
    nmb::noteLaunch();
    first = false;
    k0 += kMaxK;
  } while (k0 < K);
  if (mode == 0 && !single) {
    nmb_contract_finish_rowcol<<<(unsigned)((M * N + 255) / 256), 256, 0, stream>>>(out, M, N, ldo, nA, nB,
                                                                                   alpha, rc.func);
    nmb::noteLaunch();
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    nmb::setError("contraction launch failed: %s", cudaGetErrorString(e));
    return false;
  }
  return true;
}

bool unitStride(const GPUXMemref2f *m) { return m->strides[0] == 1 || m->strides[1] == 1; }

} // namespace

namespace {
// Enqueues C = alpha * A @ B + beta * C on the queue's stream.
bool enqueueGemm(void *queue, const GPUXMemref2f *a, const GPUXMemref2f *b, float alpha, float beta,
                 GPUXMemref2f *c) {
  if (!queue || !a || !b || !c) {
    nmb::setError("mkl_gemm_float32_device: null argument");
    return false;
  }
  const GPUXMemref2f *ops[3] = {a, b, c};
  const char names[3] = {'a', 'b', 'c'};
  for (int i = 0; i < 3; ++i)
    if (!unitStride(ops[i]) && ops[i]->dims[0] > 1 && ops[i]->dims[1] > 1) {
      // NumpyLinalg.cpp:73-86
      nmb::setError("mkl gemm suports only arrays contiguous on inner dimension; '%c' strides "
                    "are %zu and %zu",
                    names[i], ops[i]->strides[0], ops[i]->strides[1]);
      return false;
    }
  if (a->dims[1] != b->dims[0] || c->dims[0] != a->dims[0] || c->dims[1] != b->dims[1]) {
    nmb::setError("mkl_gemm_float32_device: shape mismatch (%zu,%zu) @ (%zu,%zu) -> (%zu,%zu)",
                  a->dims[0], a->dims[1], b->dims[0], b->dims[1], c->dims[0], c->dims[1]);
    return false;
  }
  const bool c_rowmajor = c->strides[1] == 1 || c->dims[1] == 1;
  Operand A{a->data + a->offset, (int64_t)a->dims[0], (int64_t)a->dims[1], (int64_t)a->strides[0],
            (int64_t)a->strides[1]};
  // rows of the second operand are the columns of b
  Operand B{b->data + b->offset, (int64_t)b->dims[1], (int64_t)b->dims[0], (int64_t)b->strides[1],
            (int64_t)b->strides[0]};
  float *out = c->data + c->offset;
  if (c_rowmajor)
    return runContraction(queue, A, B, out, (int64_t)c->strides[0], 1, alpha, beta);
  // column-major C: compute C^T = B^T . A^T, which is row-major
  return runContraction(queue, B, A, out, (int64_t)c->strides[1], 1, alpha, beta);
}
} // namespace

// C = alpha * A @ B + beta * C (NumpyLinalg.cpp:67-147); blocking like the
// reference's `.wait()`.
GPUX_EXPORT void _mlir_ciface_mkl_gemm_float32_device(void *queue, const GPUXMemref2f *a,
                                                      const GPUXMemref2f *b, float alpha,
                                                      float beta, GPUXMemref2f *c) {
  if (!enqueueGemm(queue, a, b, alpha, beta, c))
    return;
  nmb::QueueView qv;
  if (nmb::queueView(queue, &qv)) {
    cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(qv.stream));
    if (e != cudaSuccess)
      nmb::setError("mkl_gemm_float32_device failed: %s", cudaGetErrorString(e));
  }
}

// The same product without the host-side wait: asynchronous on the queue's
// stream (so it can be recorded in a CUDA graph); returns an event.
GPUX_EXPORT void *_mlir_ciface_nmb_gemm_float32_device_async(void *queue, const GPUXMemref2f *a,
                                                             const GPUXMemref2f *b, float alpha,
                                                             float beta, GPUXMemref2f *c) {
  if (!enqueueGemm(queue, a, b, alpha, beta, c))
    return nullptr;
  return nmb::recordEventOn(queue);
}

GPUX_EXPORT void mkl_gemm_float32_device(void *q, const GPUXMemref2f *a, const GPUXMemref2f *b,
                                         float alpha, float beta, GPUXMemref2f *c) {
  _mlir_ciface_mkl_gemm_float32_device(q, a, b, alpha, beta, c);
}

GPUX_EXPORT void *_mlir_ciface_nmb_pairwise_distance_float32_device(void *queue,
                                                                    const GPUXMemref2f *x,
                                                                    const GPUXMemref2f *y,
                                                                    GPUXMemref2f *d) {
  if (!queue || !x || !y || !d) {
    nmb::setError("nmb_pairwise_distance_float32_device: null argument");
    return nullptr;
  }
  if (x->dims[1] != y->dims[1] || d->dims[0] != x->dims[0] || d->dims[1] != y->dims[0]) {
    nmb::setError("nmb_pairwise_distance_float32_device: shape mismatch x (%zu,%zu), y (%zu,%zu), "
                  "d (%zu,%zu)",
                  x->dims[0], x->dims[1], y->dims[0], y->dims[1], d->dims[0], d->dims[1]);
    return nullptr;
  }
  if (d->strides[1] != 1 && d->dims[1] > 1) {
    nmb::setError("nmb_pairwise_distance_float32_device: d must be row-major");
    return nullptr;
  }
  Operand X{x->data + x->offset, (int64_t)x->dims[0], (int64_t)x->dims[1], (int64_t)x->strides[0],
            (int64_t)x->strides[1]};
  Operand Y{y->data + y->offset, (int64_t)y->dims[0], (int64_t)y->dims[1], (int64_t)y->strides[0],
            (int64_t)y->strides[1]};
  RowCol rc;
  rc.rowKind = rc.colKind = kTermNorms;
  rc.func = 1;
  if (!runContraction(queue, X, Y, d->data + d->offset, (int64_t)d->strides[0], 0, -2.f, 0.f, rc))
    return nullptr;
  return nmb::recordEventOn(queue);
}

// d[i, j] = func(alpha * sum_k x[i, k] y[j, k] + row term[i] + column term[j]):
// the contraction with the elementwise chain around the product run as its
// epilogue.  Term kinds: 0 none, 1 the squared norms of the operand's rows
// (taken from the packing prepass), 2 a contiguous float32 vector of M (row) or
// N (column) values.  func: 0 identity, 1 sqrt(max(., 0)).
GPUX_EXPORT void *_mlir_ciface_nmb_contract_rowcol_float32_device(
    void *queue, const GPUXMemref2f *x, const GPUXMemref2f *y, float alpha, int rowKind, const float *rowv,
    int colKind, const float *colv, int func, GPUXMemref2f *d) {
  if (!queue || !x || !y || !d) {
    nmb::setError("nmb_contract_rowcol_float32_device: null argument");
    return nullptr;
  }
  if (x->dims[1] != y->dims[1] || d->dims[0] != x->dims[0] || d->dims[1] != y->dims[0]) {
    nmb::setError("nmb_contract_rowcol_float32_device: shape mismatch x (%zu,%zu), y (%zu,%zu), "
                  "d (%zu,%zu)",
                  x->dims[0], x->dims[1], y->dims[0], y->dims[1], d->dims[0], d->dims[1]);
    return nullptr;
  }
  if (d->strides[1] != 1 && d->dims[1] > 1) {
    nmb::setError("nmb_contract_rowcol_float32_device: d must be row-major");
    return nullptr;
  }
  if (rowKind < 0 || rowKind > 2 || colKind < 0 || colKind > 2 || func < 0 || func > 1 ||
      (rowKind == kTermVector && !rowv) || (colKind == kTermVector && !colv)) {
    nmb::setError("nmb_contract_rowcol_float32_device: bad term kind or function");
    return nullptr;
  }
  Operand X{x->data + x->offset, (int64_t)x->dims[0], (int64_t)x->dims[1], (int64_t)x->strides[0],
            (int64_t)x->strides[1]};
  Operand Y{y->data + y->offset, (int64_t)y->dims[0], (int64_t)y->dims[1], (int64_t)y->strides[0],
            (int64_t)y->strides[1]};
  RowCol rc;
  rc.rowKind = rowKind;
  rc.colKind = colKind;
  rc.rowv = rowv;
  rc.colv = colv;
  rc.func = func;
  if (!runContraction(queue, X, Y, d->data + d->offset, (int64_t)d->strides[0], 0, alpha, 0.f, rc))
    return nullptr;
  return nmb::recordEventOn(queue);
}
