/*
 * C-ABI of libnumba_mlir_gpu_runtime_cuda.so -- the CUDA (sm_100a) replacement
 * for numba-mlir's SYCL GPU runtime.
 *
 * Every symbol has C linkage, takes plain pointers and sizes, and is what the
 * JIT-generated host code of numba-mlir binds by name (the reference registers
 * these names in numba_mlir/numba_mlir/mlir/gpu_runtime.py:34-81 and emits the
 * calls in mlir/lib/Conversion/GpuRuntimeToLlvm.cpp:95-194).  Each declaration
 * cites the reference definition it replaces.
 *
 * Error model.  The reference prints to stdout and abort()s on any failure
 * (numba_mlir_gpu_runtime_sycl/lib/Utils.hpp:8-21).  This library records the
 * message in a sticky per-process slot (gpuxGetLastError), prints it to stderr
 * and returns NULL / does nothing; set NUMBA_MLIR_GPU_RUNTIME_ABORT=1 to get
 * the reference's abort() behaviour.
 */
#ifndef NUMBA_MLIR_GPU_RUNTIME_CUDA_H
#define NUMBA_MLIR_GPU_RUNTIME_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- shared types: numba_mlir_gpu_common/GpuCommon.hpp:30-64 ------------- */

/* GpuAllocType, GpuCommon.hpp:30 */
enum {
  GPUX_ALLOC_DEVICE = 0,
  GPUX_ALLOC_SHARED = 1,
  GPUX_ALLOC_LOCAL = 2,
  GPUX_ALLOC_HOST = 3
};

/* GpuParamType, GpuCommon.hpp:32-42 */
enum {
  GPUX_PARAM_NULL = 0,
  GPUX_PARAM_BOOL = 1,
  GPUX_PARAM_INT8 = 2,
  GPUX_PARAM_INT16 = 3,
  GPUX_PARAM_INT32 = 4,
  GPUX_PARAM_INT64 = 5,
  GPUX_PARAM_FLOAT32 = 6,
  GPUX_PARAM_FLOAT64 = 7,
  GPUX_PARAM_PTR = 8
};

/* GPUParamDesc, GpuCommon.hpp:45-55: `data` points AT the argument value.
 * A GPUX_PARAM_PTR entry with data == NULL asks for `size` bytes of
 * work-group-local memory; the kernel receives, in that pointer-sized slot,
 * the byte offset of the region inside its dynamic shared memory.
 * The array is terminated by {NULL, 0, GPUX_PARAM_NULL}. */
typedef struct GPUXParamDesc {
  const void *data;
  int32_t size;
  int32_t type;
} GPUXParamDesc;

/* GPUAllocResult, GpuCommon.hpp:61-64 */
typedef struct GPUXAllocResult {
  void *ptr;
  void *event;
} GPUXAllocResult;

/* Memref<2,T>, numba_mlir/numba_mlir/math_runtime/include/Common.hpp:17-23.
 * dims and strides are in ELEMENTS. */
typedef struct GPUXMemref2f {
  void *userData;
  float *data;
  size_t offset;
  size_t dims[2];
  size_t strides[2];
} GPUXMemref2f;
typedef struct GPUXMemref2d {
  void *userData;
  double *data;
  size_t offset;
  size_t dims[2];
  size_t strides[2];
} GPUXMemref2d;

/* ---- the 13 reference exports -------------------------------------------- */

/* numba_mlir_gpu_runtime_sycl/lib/GpuRuntime.cpp:361.  deviceName: NULL or ""
 * (-> $NUMBA_MLIR_DEFAULT_DEVICE, else device 0), "cuda", "cuda:N",
 * "cuda:gpu:N", "gpu:N" or "N".  The queue is refcounted; buffers and events
 * created from it keep it alive (GpuRuntime.cpp:248-260,287-300). */
void *gpuxQueueCreate(const char *deviceName);
/* GpuRuntime.cpp:367 */
void gpuxQueueDestroy(void *queue);
/* GpuRuntime.cpp:373.  The blob is one of: an sm_100a cubin / fatbin, PTX
 * text, CUDA C source prefixed by the line "//NMB200:CUDA-SOURCE" (compiled
 * with NVRTC for sm_100a, the analogue of the driver JIT the reference gets
 * from zeModuleCreate on SPIR-V), or the text "NMB200:BUILTIN" which names the
 * hand-written kernels linked into this library. */
void *gpuxModuleLoad(void *queue, const void *data, size_t dataSize);
/* GpuRuntime.cpp:379 */
void gpuxModuleDestroy(void *module);
/* GpuRuntime.cpp:385 */
void *gpuxKernelGet(void *module, const char *name);
/* GpuRuntime.cpp:393 */
void gpuxKernelDestroy(void *kernel);
/* GpuRuntime.cpp:399.  grid* are group counts, block* group sizes; events is
 * a NULL-terminated array of event handles; params a GPUXParamDesc array.
 * Returns an event to pass to gpuxWait / gpuxDestroyEvent. */
void *gpuxLaunchKernel(void *queue, void *kernel, size_t gridX, size_t gridY,
                       size_t gridZ, size_t blockX, size_t blockY,
                       size_t blockZ, void *events, void *params);
/* Addition (no reference counterpart): gpuxLaunchKernel without the event, for
 * callers that order their work by the queue alone and would destroy the
 * event at once (saves the event record per launch).  Returns 1, or 0 with
 * the error set. */
int gpuxLaunchKernelNoEvent(void *queue, void *kernel, size_t gridX,
                            size_t gridY, size_t gridZ, size_t blockX,
                            size_t blockY, size_t blockZ, void *events,
                            void *params);
/* GpuRuntime.cpp:412.  Blocks until the event is reached.  With the
 * environment variable NUMBA_MLIR_GPU_WAIT_TIMEOUT_MS set to a positive number
 * the wait is bounded on the host: past that many milliseconds the call
 * returns with the error set (gpuxGetLastError) and the device work is left
 * running.  NUMBA_MLIR_GPU_RUNTIME_NVTX=1 wraps every gpux* call in an NVTX
 * range of its name; NUMBA_MLIR_LOG_GPU_RUNTIME_CALLS=1 prints the
 * reference's enter/exit lines (GpuRuntime.cpp:29-35,61-82). */
void gpuxWait(void *queue, void *event);
/* GpuRuntime.cpp:419 */
void gpuxDestroyEvent(void *queue, void *event);
/* GpuRuntime.cpp:427.  type is a GPUX_ALLOC_* value; LOCAL yields ptr NULL. */
void gpuxAlloc(void *queue, size_t size, size_t alignment, int type,
               void *events, GPUXAllocResult *ret);
/* GpuRuntime.cpp:439 */
void gpuxDeAlloc(void *queue, void *ptr);
/* GpuRuntime.cpp:445, heuristic of GpuModule.cpp:453-509: gridSize holds the
 * GLOBAL sizes; dimensions of size <= 1 get block size 1. */
void gpuxSuggestBlockSize(void *queue, void *kernel, const uint32_t *gridSize,
                          uint32_t *blockSize, size_t numDims);
/* GpuRuntime.cpp:455.  The reference copies a native sycl::queue; here the
 * native handle is a cudaStream_t (NULL = the legacy default stream) of the
 * current device and the result is a queue handle that launches on it. */
void *gpuxDuplicateQueue(void *nativeStream);

/* Device BLAS entry: math_runtime/sycl/lib/NumpyLinalg.cpp:166-175, bound as
 * "_mlir_ciface_mkl_gemm_float32_device" (mlir/math_runtime.py:20-40).
 * C = alpha * A @ B + beta * C; every operand needs one unit stride
 * (NumpyLinalg.cpp:73-86).  Blocking, like the reference's .wait(). */
void _mlir_ciface_mkl_gemm_float32_device(void *queue, const GPUXMemref2f *a,
                                          const GPUXMemref2f *b, float alpha,
                                          float beta, GPUXMemref2f *c);
void mkl_gemm_float32_device(void *queue, const GPUXMemref2f *a,
                             const GPUXMemref2f *b, float alpha, float beta,
                             GPUXMemref2f *c);
/* The float64 variant the reference registers beside it
 * (mlir/math_runtime.py:36-40): any strides, blocking. */
void _mlir_ciface_mkl_gemm_float64_device(void *queue, const GPUXMemref2d *a,
                                          const GPUXMemref2d *b, double alpha,
                                          double beta, GPUXMemref2d *c);
void mkl_gemm_float64_device(void *queue, const GPUXMemref2d *a,
                             const GPUXMemref2d *b, double alpha, double beta,
                             GPUXMemref2d *c);

/* ---- extensions (no counterpart in the reference, where dpctl moved the
 * data: mlir/tests/test_gpu.py:52-87) ------------------------------------- */

enum { GPUX_COPY_H2D = 0, GPUX_COPY_D2H = 1, GPUX_COPY_D2D = 2, GPUX_COPY_DEFAULT = 3 };
/* Asynchronous copy on the queue's stream; returns an event. */
void *gpuxMemcpy(void *queue, void *dst, const void *src, size_t bytes,
                 int kind, void *events);
/* Asynchronous byte fill on the queue's stream; returns an event. */
void *gpuxMemset(void *queue, void *dst, int value, size_t bytes, void *events);
/* Records an event at the current tail of the queue's stream. */
void *gpuxRecordEvent(void *queue);
/* Orders everything submitted to the queue from now on after the events of a
 * NULL-terminated Event*[] (events of other queues of the same device become
 * stream dependencies; nothing blocks on the host).  Returns 0 on success.
 * The launch, alloc, memcpy and memset entries take the same kind of list;
 * this entry is for callers that submit through a layer which does not pass
 * one on.  No counterpart in the reference, whose host code waits on every
 * event (GpuRuntimeToLlvm.cpp:619-622). */
int gpuxQueueWaitEvents(void *queue, void *events);
/* Orders everything submitted to the queue from now on after the work already
 * submitted to another CUDA stream of the same device (cudaStream_t; NULL, 1
 * and 2 name the default streams as in the CUDA array interface).  This is how
 * an array imported from another library is consumed on the producer's terms:
 * version 3 of __cuda_array_interface__ carries the stream the data is ready
 * on.  Returns 0 on success.  No counterpart in the reference, where dpctl
 * owns the queues of imported arrays. */
int gpuxQueueWaitStream(void *queue, void *nativeStream);
/* Memory that the other GPU processes of the box can map (one process per
 * GPU): gpuxPeerAlloc returns zero-filled device memory outside the
 * stream-ordered pool, gpuxPeerExport writes an opaque handle of
 * GPUX_PEER_HANDLE_BYTES bytes that another process passes to gpuxPeerOpen to
 * obtain the address of the same memory in its own address space (peer access
 * over NVLink is enabled on first use), gpuxPeerClose unmaps it and
 * gpuxPeerFree releases the owner's allocation.  Export and open return 0 /
 * non-NULL on success.  They carry the mailboxes of the small all-reduce
 * between shards; no counterpart in the reference, which drives one device
 * per process and has no exchange between devices. */
#define GPUX_PEER_HANDLE_BYTES 64
void *gpuxPeerAlloc(void *queue, size_t size);
void gpuxPeerFree(void *queue, void *ptr);
int gpuxPeerExport(void *ptr, void *handle);
void *gpuxPeerOpen(void *queue, const void *handle);
void gpuxPeerClose(void *queue, void *ptr);
/* Milliseconds between two completed events of the same device. */
float gpuxEventElapsedMs(void *startEvent, void *endEvent);
/* Blocks until everything submitted to the queue has finished. */
void gpuxQueueSynchronize(void *queue);
/* cudaStream_t of the queue (role of GPUQueueInterface::getQueue,
 * GpuCommon.hpp:25-27) and its CUDA device ordinal. */
void *gpuxQueueGetStream(void *queue);
int gpuxQueueGetDevice(void *queue);
/* Multiprocessor count of the queue's device (-1 on error); launch shapes are
 * sized in multiples of it. */
int gpuxQueueGetSmCount(void *queue);
/* Device address of a 4-byte status word owned by the queue.  Kernels of this
 * library bound every device-side wait; one that gives up stores a non-zero
 * code here instead of hanging.  Read it back with gpuxMemcpy. */
void *gpuxQueueStatusPtr(void *queue);
/* Sticky error message of the last failed call (NULL when none). */
const char *gpuxGetLastError(void);
void gpuxClearLastError(void);
/* Number of kernels launched by this library since load (all queues). */
uint64_t gpuxLaunchCount(void);
/* Test hook, host side only: the next `count` calls this library makes to the
 * CUDA driver entry point `name` ("cuLaunchKernel", "cuModuleLoadDataEx",
 * "cuModuleGetFunction") return the CUresult `code` without reaching the
 * driver; count 0 clears a pending injection.  The reference has no such
 * hook; its failures abort (numba_mlir_gpu_runtime_sycl/lib/Utils.hpp:8-21). */
void gpuxTestInjectDriverFault(const char *name, int code, int count);

/* CUDA graphs: gpuxGraphBegin starts recording everything submitted to the
 * queue (nothing runs), gpuxGraphEnd returns a replayable graph handle,
 * gpuxGraphLaunch replays it on the queue's stream and returns an event.
 * Events returned by launches made while recording must only be destroyed,
 * not waited on.  Do not allocate or free between Begin and End. */
void gpuxGraphBegin(void *queue);
void *gpuxGraphEnd(void *queue);
void *gpuxGraphLaunch(void *queue, void *graph);
void gpuxGraphDestroy(void *graph);

/* Host-only: NVRTC-compiles a "//NMB200:CUDA-SOURCE" blob to an sm_100a cubin
 * without touching a device; the result is malloc()ed, release it with
 * gpuxFreeHostBlob. */
void *gpuxCompileToCubin(const void *data, size_t dataSize, size_t *outSize);
void gpuxFreeHostBlob(void *blob);
/* '\n'-separated names of the kernels behind the "NMB200:BUILTIN" module. */
const char *gpuxBuiltinKernelNames(void);

/* Library routine surfaced the way the reference surfaces device library
 * calls (external_call + "gpu_runtime.device_func",
 * mlir/numpy/funcs.py:780-785): D[i,j] = sqrt(max(|x_i|^2 + |y_j|^2 -
 * 2 x_i.y_j, 0)) with the dot products on tcgen05 tensor cores (3xTF32).
 * Semantics follow the reference's pairwise kernels
 * (mlir/tests/test_gpu.py:1396-1430,2226-2266).  x: (M,K), y: (N,K),
 * d: (M,N), row-major float32 with unit inner stride.  Asynchronous on the
 * queue's stream; returns an event. */
void *_mlir_ciface_nmb_pairwise_distance_float32_device(void *queue,
                                                        const GPUXMemref2f *x,
                                                        const GPUXMemref2f *y,
                                                        GPUXMemref2f *d);

/* The product of mkl_gemm_float32_device without its host-side wait
 * (NumpyLinalg.cpp:143-146 waits on the oneMKL event): asynchronous on the
 * queue's stream, so a step that contains it can be recorded with
 * gpuxGraphBegin/End; returns an event. */
void *_mlir_ciface_nmb_gemm_float32_device_async(void *queue, const GPUXMemref2f *a,
                                                 const GPUXMemref2f *b, float alpha,
                                                 float beta, GPUXMemref2f *c);
void *_mlir_ciface_nmb_gemm_float64_device_async(void *queue, const GPUXMemref2d *a,
                                                 const GPUXMemref2d *b, double alpha,
                                                 double beta, GPUXMemref2d *c);

/* The contraction with the elementwise chain around the product fused as its
 * epilogue, what the reference gets by fusing the linalg.generic ops around a
 * device library call (external_call + "gpu_runtime.device_func",
 * mlir/numpy/funcs.py:780-785):
 *   d[i,j] = func(alpha * sum_k x[i,k] y[j,k] + row[i] + col[j])
 * x: (M,K), y: (N,K), d: (M,N) row-major float32.  rowKind / colKind: 0 no
 * term, 1 the squared norms of the operand's rows (taken from the packing
 * prepass; rowv / colv ignored), 2 a contiguous float32 device vector of M
 * (rowv) or N (colv) values.  func: 0 identity, 1 sqrt(max(., 0)).  The
 * pairwise distance above is alpha = -2, both kinds 1, func 1.  Asynchronous
 * on the queue's stream; returns an event. */
void *_mlir_ciface_nmb_contract_rowcol_float32_device(void *queue, const GPUXMemref2f *x,
                                                      const GPUXMemref2f *y, float alpha,
                                                      int rowKind, const float *rowv,
                                                      int colKind, const float *colv, int func,
                                                      GPUXMemref2f *d);

/* No counterpart in the reference.  *out = sum of data[0..n) accumulated in
 * int64, like the full integer reduction above, for callers that must not
 * allocate: a thread that may not wait on the CUDA allocator (a monitor or a
 * real-time loop with a latency budget), a process whose device memory was all
 * handed out at start-up.  The kernel's scratch lives in an 8 KB array inside
 * the library image (held by every GPU that loads the library until exit), so
 * the call makes no device allocation and, on its success path, no host
 * allocation (it takes one short mutex; only the error path formats a
 * message); it runs asynchronously on the queue's stream.
 * data must be 16-byte aligned, 1 <= n <= 2^32; anything else is refused with
 * an error (non-zero return, gpuxGetLastError).  All calls on a device share
 * the array: calls that overlap on the GPU race, so keep them on one stream.
 * The first call on each device also resolves the array's device address;
 * make it before any stream capture.
 * Every wait inside the kernel is bounded.  A call whose wait ran out leaves
 * *out untouched and sets a status word in the array that only
 * gpuxSumInt32NoAllocStatus reports (the queue's own status word is not
 * involved). */
int gpuxSumInt32NoAlloc(void *queue, const int32_t *data, size_t n, int64_t *out);

/* No counterpart in the reference.  Failure report of gpuxSumInt32NoAlloc:
 * waits for the queue's stream, then returns 0 when every call issued so far
 * on the queue's device completed, 1 when a bounded wait inside one of them
 * ran out (that call did not write *out), -1 on a CUDA error
 * (gpuxGetLastError).  A non-zero status is cleared by being read.  Allocates
 * nothing: the word is read with a 4-byte copy into a local variable. */
int gpuxSumInt32NoAllocStatus(void *queue);

#ifdef __cplusplus
}
#endif
#endif /* NUMBA_MLIR_GPU_RUNTIME_CUDA_H */
