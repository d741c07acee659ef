// Internal mirror of the shared types of the gpux* C-ABI, with the layout
// assumptions the reference compiler bakes into generated host code
// (mlir/lib/Conversion/GpuRuntimeToLlvm.cpp:87-93 mirrors GPUParamDesc as the
// LLVM literal struct {ptr, i32, i32}) checked at compile time.
#pragma once

#include "../../include/numba_mlir_gpu_runtime_cuda.h"

#include <cstddef>
#include <cstdint>

static_assert(sizeof(GPUXParamDesc) == 16, "GPUParamDesc must be {ptr,i32,i32}");
static_assert(offsetof(GPUXParamDesc, size) == 8, "GPUParamDesc.size offset");
static_assert(offsetof(GPUXParamDesc, type) == 12, "GPUParamDesc.type offset");
static_assert(sizeof(GPUXAllocResult) == 16, "GPUAllocResult must be {ptr,ptr}");
static_assert(sizeof(GPUXMemref2f) == 56, "Memref<2,float> layout");

namespace nmb {

// One hand-written kernel linked into the library and reachable through
// gpuxModuleLoad("NMB200:BUILTIN") + gpuxKernelGet(name).
struct BuiltinKernel {
  const char *name;
  const void *hostFunc; // address of the __global__ function's host stub
  int dynSmemBytes;     // dynamic shared memory the kernel itself needs
};

void registerBuiltin(const char *name, const void *hostFunc, int dynSmemBytes);

struct BuiltinRegistrar {
  BuiltinRegistrar(const char *name, const void *hostFunc, int dynSmemBytes) {
    registerBuiltin(name, hostFunc, dynSmemBytes);
  }
};

// Internal launch helpers used by the library routines (gemm, pairwise).
struct QueueView {
  void *stream; // cudaStream_t
  int device;
};
bool queueView(void *queue, QueueView *out);
void *recordEventOn(void *queue);           // event at the stream tail
void setError(const char *fmt, ...);        // sticky error + stderr
void noteLaunch();                          // bumps gpuxLaunchCount
void *scratchGet(void *queue, size_t bytes); // per-queue grow-only scratch
uint32_t *statusWord(void *queue);            // per-queue device word set by timed-out waits

} // namespace nmb

#define NMB_REGISTER_KERNEL(fn, smem)                                          \
  static ::nmb::BuiltinRegistrar nmb_registrar_##fn(#fn, (const void *)(fn), (smem))
