/* The call sequence the reference's generated host code makes for one offloaded
 * loop (mlir/lib/Conversion/GpuRuntimeToLlvm.cpp:228-857), written against
 * include/numba_mlir_gpu_runtime_cuda.h in plain C: create a queue, allocate,
 * load a module, get a kernel, launch it from a GPUParamDesc array that ends
 * with {NULL, 0, null}, wait, release everything.  The kernel is the library's
 * built-in broadcast add (out = a + b[i % inner]).
 *
 *   host_example            full run on the first CUDA device; prints "ok"
 *   host_example --no-device  only the calls that need no device (error paths)
 */
#include "numba_mlir_gpu_runtime_cuda.h"

#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define CHECK(cond, what)                                                         \
  do {                                                                            \
    if (!(cond)) {                                                                \
      const char *e = gpuxGetLastError();                                         \
      fprintf(stderr, "FAILED: %s (%s)\n", what, e ? e : "no error text");        \
      return 1;                                                                   \
    }                                                                             \
  } while (0)

int main(int argc, char **argv) {
  if (argc > 1 && strcmp(argv[1], "--no-device") == 0) {
    gpuxClearLastError();
    CHECK(gpuxGetLastError() == NULL, "no sticky error after clearing");
    CHECK(gpuxModuleLoad(NULL, "x", 1) == NULL, "module load without a queue is refused");
    CHECK(gpuxGetLastError() != NULL, "the refusal left a message");
    CHECK(strstr(gpuxBuiltinKernelNames(), "nmb_bcast_add_f32") != NULL, "built-in kernel table");
    printf("ok (no device)\n");
    return 0;
  }

  enum { ROWS = 300, INNER = 1024, N = ROWS * INNER };
  void *queue = gpuxQueueCreate(NULL);
  CHECK(queue, "gpuxQueueCreate");

  GPUXAllocResult a, b, out;
  gpuxAlloc(queue, N * sizeof(float), 64, GPUX_ALLOC_DEVICE, NULL, &a);
  gpuxAlloc(queue, INNER * sizeof(float), 64, GPUX_ALLOC_DEVICE, NULL, &b);
  gpuxAlloc(queue, N * sizeof(float), 64, GPUX_ALLOC_DEVICE, NULL, &out);
  CHECK(a.ptr && b.ptr && out.ptr, "gpuxAlloc");
  gpuxWait(queue, a.event);
  gpuxWait(queue, b.event);
  gpuxWait(queue, out.event);
  gpuxDestroyEvent(queue, a.event);
  gpuxDestroyEvent(queue, b.event);
  gpuxDestroyEvent(queue, out.event);

  float *ha = malloc(N * sizeof(float)), *hb = malloc(INNER * sizeof(float)), *ho = malloc(N * sizeof(float));
  for (int i = 0; i < N; ++i)
    ha[i] = (float)(i % 977) * 0.25f;
  for (int i = 0; i < INNER; ++i)
    hb[i] = (float)i - 512.f;
  void *ev = gpuxMemcpy(queue, a.ptr, ha, N * sizeof(float), GPUX_COPY_H2D, NULL);
  CHECK(ev, "gpuxMemcpy a");
  gpuxDestroyEvent(queue, ev);
  ev = gpuxMemcpy(queue, b.ptr, hb, INNER * sizeof(float), GPUX_COPY_H2D, NULL);
  CHECK(ev, "gpuxMemcpy b");
  gpuxDestroyEvent(queue, ev);

  static const char blob[] = "NMB200:BUILTIN";
  void *module = gpuxModuleLoad(queue, blob, sizeof(blob) - 1);
  CHECK(module, "gpuxModuleLoad");
  void *kernel = gpuxKernelGet(module, "nmb_bcast_add_f32");
  CHECK(kernel, "gpuxKernelGet");

  int64_t n = N, inner = INNER;
  GPUXParamDesc params[] = {
      {&a.ptr, sizeof(void *), GPUX_PARAM_PTR},   {&b.ptr, sizeof(void *), GPUX_PARAM_PTR},
      {&out.ptr, sizeof(void *), GPUX_PARAM_PTR}, {&n, sizeof(n), GPUX_PARAM_INT64},
      {&inner, sizeof(inner), GPUX_PARAM_INT64},  {NULL, 0, GPUX_PARAM_NULL},
  };
  const size_t tile = 256 * 4 * 4; /* elements per group of this kernel */
  ev = gpuxLaunchKernel(queue, kernel, (N + tile - 1) / tile, 1, 1, 256, 1, 1, NULL, params);
  CHECK(ev, "gpuxLaunchKernel");
  gpuxWait(queue, ev);
  gpuxDestroyEvent(queue, ev);

  ev = gpuxMemcpy(queue, ho, out.ptr, N * sizeof(float), GPUX_COPY_D2H, NULL);
  CHECK(ev, "gpuxMemcpy out");
  gpuxWait(queue, ev);
  gpuxDestroyEvent(queue, ev);
  for (int i = 0; i < N; ++i)
    if (ho[i] != ha[i] + hb[i % INNER]) {
      fprintf(stderr, "FAILED: element %d is %g, expected %g\n", i, ho[i], ha[i] + hb[i % INNER]);
      return 1;
    }

  gpuxKernelDestroy(kernel);
  gpuxModuleDestroy(module);
  gpuxDeAlloc(queue, a.ptr);
  gpuxDeAlloc(queue, b.ptr);
  gpuxDeAlloc(queue, out.ptr);
  gpuxQueueDestroy(queue);
  free(ha);
  free(hb);
  free(ho);
  printf("ok: %d elements through the C ABI, %llu launch(es)\n", (int)N, (unsigned long long)gpuxLaunchCount());
  return 0;
}
