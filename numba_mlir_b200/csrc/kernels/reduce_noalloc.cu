// gpuxSumInt32NoAlloc: the full int32 -> int64 sum for callers that cannot
// allocate device memory.
//
// Who cannot allocate: a thread that must not wait on the CUDA allocator (a
// monitor with a latency budget, a real-time loop), or a process whose device
// memory was handed out in full at start-up, so that any later allocation
// fails.  The other entry points of this library reach the same kernel through
// per-queue scratch memory that grows on demand; this one keeps its scratch
// (CTA partials, the ticket counter, the status word) in a fixed array that is
// part of the library image, so a call makes no device allocation and no host
// allocation on its success path (it takes one short mutex; only the error
// path formats a message).
//
// The cost: every GPU that loads the library holds the 8 KB array until the
// process exits, every call on a device shares it (two calls that overlap on
// the GPU, e.g. from two streams, race on it -- serialise them), and it keeps
// whatever the last call left, so each call clears the ticket counter before
// launching.  The status word is the exception: it stays set until
// gpuxSumInt32NoAllocStatus has reported it.

#include "../gpu_common.h"
#include "reduce_common.cuh"

#include <cuda_runtime.h>

#include <mutex>

#define GPUX_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

constexpr int kMaxCtas = 444;                // three 65 KB CTAs per SM on 148 SMs
constexpr size_t kPartialBytes = 7168;       // kMaxCtas int64 partials, rounded up
constexpr size_t kCounterOffset = kPartialBytes;        // one ticket counter
constexpr size_t kStatusOffset = kPartialBytes + 256;   // one status word
constexpr size_t kScratchBytes = 8192;
constexpr uint64_t kMaxElements = 1ull << 32; // stated limit of this entry point

// Scratch of the no-allocation entry point.  In host code this name is only a
// handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

using SumI32 = nmb::red::SumR<int32_t>;

extern "C" __global__ void __launch_bounds__(nmb::red::kThreads, 3)
    nmb_noalloc_sum_i32(const int32_t *a, int64_t *out, unsigned char *scratch, int64_t n,
                        int64_t span) {
  extern __shared__ __align__(128) unsigned char nmb_smem[];
  // GuardOut: a call whose bounded wait ran out leaves *out untouched
  nmb::red::reduce_all_body<SumI32, true>(a, out, reinterpret_cast<int64_t *>(scratch),
                                    reinterpret_cast<uint32_t *>(scratch + kCounterOffset), n, span,
                                    reinterpret_cast<uint32_t *>(scratch + kStatusOffset), nmb_smem);
}

struct DeviceSetup {
  unsigned char *scratch = nullptr; // device address of g_noalloc_scratch on this device
  bool ready = false;
};
std::mutex gSetupMutex;
DeviceSetup gSetup[64];

// Resolves the array's device address once per device (that device current).
bool setupDevice(int device, DeviceSetup **out) {
  if (device < 0 || device >= 64) {
    nmb::setError("gpuxSumInt32NoAlloc: device index %d not supported", device);
    return false;
  }
  DeviceSetup &dev = gSetup[device];
  std::lock_guard<std::mutex> lock(gSetupMutex);
  if (!dev.ready) {
    void *ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || !ptr) {
      nmb::setError("gpuxSumInt32NoAlloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      (void)cudaGetLastError();
      return false;
    }
    e = cudaFuncSetAttribute(nmb_noalloc_sum_i32, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             nmb::red::kSmemBytes);
    if (e != cudaSuccess) {
      nmb::setError("gpuxSumInt32NoAlloc: cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
      (void)cudaGetLastError();
      return false;
    }
    dev.scratch = static_cast<unsigned char *>(ptr);
    dev.ready = true;
  }
  *out = &dev;
  return true;
}

} // namespace

// Returns 0 on success.  The first call on each device resolves the device
// address of the scratch array and raises the kernel's shared-memory limit;
// make that first call outside any stream capture.
GPUX_EXPORT int gpuxSumInt32NoAlloc(void *queue, const int32_t *data, size_t n, int64_t *out) {
  if (!queue || !out || (!data && n)) {
    nmb::setError("gpuxSumInt32NoAlloc: null argument");
    return 1;
  }
  if (n == 0 || n > kMaxElements) {
    nmb::setError("gpuxSumInt32NoAlloc: n = %zu is outside 1 .. 2^32 elements, the range this "
                  "entry point is built for",
                  n);
    return 1;
  }
  if (reinterpret_cast<uintptr_t>(data) % 16 != 0 || reinterpret_cast<uintptr_t>(out) % 8 != 0) {
    nmb::setError("gpuxSumInt32NoAlloc: data must be 16-byte aligned and out 8-byte aligned");
    return 1;
  }
  nmb::QueueView qv;
  if (!nmb::queueView(queue, &qv)) // also makes the queue's device current
    return 1;
  cudaStream_t stream = static_cast<cudaStream_t>(qv.stream);
  DeviceSetup *devp = nullptr;
  if (!setupDevice(qv.device, &devp))
    return 1;
  DeviceSetup &dev = *devp;
  // The array keeps the previous call's contents: the ticket counter must start
  // at zero (the partials are fully rewritten).  The status word is left alone:
  // it belongs to gpuxSumInt32NoAllocStatus.
  cudaError_t e = cudaMemsetAsync(dev.scratch + kCounterOffset, 0, kStatusOffset - kCounterOffset, stream);
  if (e != cudaSuccess) {
    nmb::setError("gpuxSumInt32NoAlloc: cudaMemsetAsync failed: %s", cudaGetErrorString(e));
    (void)cudaGetLastError();
    return 1;
  }
  const int64_t tile = nmb::red::kTileBytes / sizeof(int32_t);
  int64_t grid = (int64_t)((n + tile - 1) / tile);
  if (grid > kMaxCtas)
    grid = kMaxCtas;
  int64_t span = ((int64_t)n + grid - 1) / grid;
  span = (span + tile - 1) / tile * tile;
  nmb_noalloc_sum_i32<<<(unsigned)grid, nmb::red::kThreads, nmb::red::kSmemBytes, stream>>>(
      data, out, dev.scratch, (int64_t)n, span);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    nmb::setError("gpuxSumInt32NoAlloc: launch failed: %s", cudaGetErrorString(e));
    return 1;
  }
  nmb::noteLaunch();
  return 0;
}

// Reports whether every gpuxSumInt32NoAlloc call issued so far on the queue's
// device ran to completion: 0 = yes; 1 = a bounded wait inside a call ran out
// (that call left *out untouched); -1 = a CUDA error (gpuxGetLastError).
// Waits for the queue's stream, reads the word with a 4-byte copy into a
// variable of its own and, when the word was set, clears it.  No allocation.
GPUX_EXPORT int gpuxSumInt32NoAllocStatus(void *queue) {
  if (!queue) {
    nmb::setError("gpuxSumInt32NoAllocStatus: null queue");
    return -1;
  }
  nmb::QueueView qv;
  if (!nmb::queueView(queue, &qv))
    return -1;
  cudaStream_t stream = static_cast<cudaStream_t>(qv.stream);
  DeviceSetup *dev = nullptr;
  if (!setupDevice(qv.device, &dev))
    return -1;
  uint32_t word = 0;
  cudaError_t e = cudaMemcpyAsync(&word, dev->scratch + kStatusOffset, sizeof(word),
                                  cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess)
    e = cudaStreamSynchronize(stream);
  if (e == cudaSuccess && word != 0)
    e = cudaMemsetAsync(dev->scratch + kStatusOffset, 0, sizeof(word), stream);
  if (e != cudaSuccess) {
    nmb::setError("gpuxSumInt32NoAllocStatus failed: %s", cudaGetErrorString(e));
    (void)cudaGetLastError();
    return -1;
  }
  return (int)word;
}
