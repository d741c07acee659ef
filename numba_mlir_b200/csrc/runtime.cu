// CUDA implementation of numba-mlir's gpux* runtime C-ABI.
//
// Replaces numba_mlir_gpu_runtime_sycl/lib/{GpuRuntime,GpuModule}.cpp: a
// refcounted queue (one CUDA stream on one device), an event free-list, device
// / managed / pinned allocation, module loading (cubin, PTX, NVRTC-compiled
// CUDA C, or the hand-written kernels linked into this library) and kernel
// launch from a GPUParamDesc array.  The driver API is reached through
// cudaGetDriverEntryPoint so the library loads on machines without a driver.

#include "gpu_common.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>
#include <dlfcn.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#define GPUX_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

// ---------------------------------------------------------------- errors ---
std::mutex gErrMutex;
std::string gLastError;
bool gHasError = false;
std::atomic<uint64_t> gLaunchCount{0};

bool envFlag(const char *name) {
  const char *v = getenv(name);
  return v && *v && strcmp(v, "0") != 0;
}

void vsetError(const char *fmt, va_list ap) {
  char buf[4096];
  vsnprintf(buf, sizeof(buf), fmt, ap);
  {
    std::lock_guard<std::mutex> g(gErrMutex);
    gLastError = buf;
    gHasError = true;
  }
  fprintf(stderr, "numba_mlir_gpu_runtime_cuda: %s\n", buf);
  fflush(stderr);
  // Reference behaviour (Utils.hpp:8-21) on request.
  if (envFlag("NUMBA_MLIR_GPU_RUNTIME_ABORT"))
    abort();
}

// Call tracing, as NUMBA_MLIR_LOG_GPU_RUNTIME_CALLS in GpuRuntime.cpp:29-35;
// NUMBA_MLIR_GPU_RUNTIME_NVTX=1 wraps every export in an NVTX range of its
// name instead (or as well), so the calls show up on a profiler's timeline.
struct FuncLog {
  const char *name;
  bool on, nvtx;
  explicit FuncLog(const char *n) : name(n) {
    static bool enabled = envFlag("NUMBA_MLIR_LOG_GPU_RUNTIME_CALLS");
    static bool ranges = envFlag("NUMBA_MLIR_GPU_RUNTIME_NVTX");
    on = enabled;
    nvtx = ranges;
    if (on) {
      fprintf(stdout, "%s enter\n", name);
      fflush(stdout);
    }
    if (nvtx)
      nvtxRangePushA(name);
  }
  ~FuncLog() {
    if (nvtx)
      nvtxRangePop();
    if (on) {
      fprintf(stdout, "%s exit\n", name);
      fflush(stdout);
    }
  }
};
#define LOG_FUNC() FuncLog _funcLog(__func__)

#define CUDA_TRY(expr, fail)                                                   \
  do {                                                                         \
    cudaError_t _e = (expr);                                                   \
    if (_e != cudaSuccess) {                                                   \
      nmb::setError("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),    \
                    __FILE__, __LINE__);                                       \
      (void)cudaGetLastError();                                                \
      fail;                                                                    \
    }                                                                          \
  } while (0)

// ------------------------------------------------------------ driver API ---
struct DriverApi {
  CUresult (*ModuleLoadDataEx)(CUmodule *, const void *, unsigned int,
                               CUjit_option *, void **) = nullptr;
  CUresult (*ModuleUnload)(CUmodule) = nullptr;
  CUresult (*ModuleGetFunction)(CUfunction *, CUmodule, const char *) = nullptr;
  CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned,
                           unsigned, unsigned, unsigned, CUstream, void **,
                           void **) = nullptr;
  CUresult (*FuncGetAttribute)(int *, CUfunction_attribute, CUfunction) = nullptr;
  CUresult (*FuncSetAttribute)(CUfunction, CUfunction_attribute, int) = nullptr;
  CUresult (*OccupancyMaxPotentialBlockSize)(int *, int *, CUfunction,
                                             CUoccupancyB2DSize, size_t,
                                             int) = nullptr;
  CUresult (*GetErrorString)(CUresult, const char **) = nullptr;
  bool ok = false;
};

DriverApi &driver() {
  static DriverApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    auto get = [](const char *name, void **fn) {
      cudaDriverEntryPointQueryResult st;
      cudaError_t e = cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &st);
      if (e != cudaSuccess || st != cudaDriverEntryPointSuccess || !*fn) {
        (void)cudaGetLastError();
        return false;
      }
      return true;
    };
    bool ok = true;
    ok &= get("cuModuleLoadDataEx", (void **)&api.ModuleLoadDataEx);
    ok &= get("cuModuleUnload", (void **)&api.ModuleUnload);
    ok &= get("cuModuleGetFunction", (void **)&api.ModuleGetFunction);
    ok &= get("cuLaunchKernel", (void **)&api.LaunchKernel);
    ok &= get("cuFuncGetAttribute", (void **)&api.FuncGetAttribute);
    ok &= get("cuFuncSetAttribute", (void **)&api.FuncSetAttribute);
    ok &= get("cuOccupancyMaxPotentialBlockSize",
              (void **)&api.OccupancyMaxPotentialBlockSize);
    ok &= get("cuGetErrorString", (void **)&api.GetErrorString);
    api.ok = ok;
  });
  return api;
}

// Host-side failure injection for tests: the next `remaining` calls of the
// named driver entry point return `code` without reaching the driver.
struct DriverFault {
  std::mutex mutex;
  std::string name;
  int code = 0;
  int remaining = 0;
};
DriverFault gDriverFault;

// True (and *out set) when the call `name` is to fail by injection.
bool injectedFault(const char *name, CUresult *out) {
  if (gDriverFault.remaining <= 0) // unlocked fast path: tests set it before the calls they aim at
    return false;
  std::lock_guard<std::mutex> g(gDriverFault.mutex);
  if (gDriverFault.remaining <= 0 || gDriverFault.name != name)
    return false;
  --gDriverFault.remaining;
  *out = static_cast<CUresult>(gDriverFault.code);
  return true;
}

// A driver call that the injection hook can replace.
#define DRV(fn, ...)                                                           \
  ([&]() -> CUresult {                                                         \
    CUresult _inj;                                                             \
    if (injectedFault("cu" #fn, &_inj))                                        \
      return _inj;                                                             \
    return driver().fn(__VA_ARGS__);                                           \
  }())

const char *cuErr(CUresult r) {
  const char *s = nullptr;
  if (driver().GetErrorString)
    driver().GetErrorString(r, &s);
  return s ? s : "unknown CUDA driver error";
}

#define CU_TRY(expr, fail)                                                     \
  do {                                                                         \
    CUresult _r = (expr);                                                      \
    if (_r != CUDA_SUCCESS) {                                                  \
      nmb::setError("%s failed: %s (%s:%d)", #expr, cuErr(_r), __FILE__,       \
                    __LINE__);                                                 \
      fail;                                                                    \
    }                                                                          \
  } while (0)

// -------------------------------------------------------- builtin kernels ---
std::vector<nmb::BuiltinKernel> &builtinTable() {
  static std::vector<nmb::BuiltinKernel> table;
  return table;
}

// ------------------------------------------------------------------ queue ---
struct Queue;

struct Event {
  cudaEvent_t ev = nullptr;
  Queue *queue = nullptr;
  Event *next = nullptr;
};

// Plays the role of numba::GPUQueueInterface (GpuCommon.hpp:18-28): the
// handle library routines receive and ask for the native stream.
struct Queue {
  std::atomic<unsigned> refcount{1};
  int device = 0;
  cudaStream_t stream = nullptr;
  bool ownsStream = true;
  std::string deviceName;

  std::mutex mutex;
  Event *freeEvents = nullptr;
  std::unordered_map<void *, int> allocs; // ptr -> GPUX_ALLOC_*
  void *scratch = nullptr;
  size_t scratchBytes = 0;
  uint32_t *status = nullptr; // device word kernels set when a bounded wait ran out

  void retain() { ++refcount; }
  void release() {
    if (--refcount == 0)
      delete this;
  }

  ~Queue() {
    cudaSetDevice(device);
    for (Event *e = freeEvents; e;) {
      Event *n = e->next;
      if (e->ev)
        cudaEventDestroy(e->ev);
      delete e;
      e = n;
    }
    if (scratch)
      cudaFreeAsync(scratch, stream);
    if (status)
      cudaFreeAsync(status, stream);
    if (ownsStream && stream) {
      cudaStreamSynchronize(stream);
      cudaStreamDestroy(stream);
    }
    (void)cudaGetLastError();
  }

  // Events keep the queue alive (GpuRuntime.cpp:272-300).
  Event *getEvent() {
    Event *e = nullptr;
    {
      std::lock_guard<std::mutex> g(mutex);
      if (freeEvents) {
        e = freeEvents;
        freeEvents = e->next;
        e->next = nullptr;
      }
    }
    if (!e) {
      e = new Event;
      e->queue = this;
      if (cudaEventCreate(&e->ev) != cudaSuccess) {
        (void)cudaGetLastError();
        delete e;
        return nullptr;
      }
    }
    retain();
    return e;
  }

  void returnEvent(Event *e) {
    {
      std::lock_guard<std::mutex> g(mutex);
      e->next = freeEvents;
      freeEvents = e;
    }
    release();
  }
};

Queue *toQueue(void *q) { return static_cast<Queue *>(q); }

bool parseDeviceIndex(const char *name, int *out) {
  // Accepted: "", "cuda", "cuda:N", "cuda:gpu:N", "gpu:N", "N".
  std::string s = name ? name : "";
  if (s.empty()) {
    const char *env = getenv("NUMBA_MLIR_DEFAULT_DEVICE");
    s = env ? env : "";
  }
  if (s.empty()) {
    // No name: the calling thread's current device, so a process that pinned
    // itself to one GPU keeps using it.
    int cur = 0;
    if (cudaGetDevice(&cur) != cudaSuccess) {
      (void)cudaGetLastError();
      cur = 0;
    }
    *out = cur;
    return true;
  }
  size_t pos = s.rfind(':');
  std::string tail = pos == std::string::npos ? s : s.substr(pos + 1);
  std::string head = pos == std::string::npos ? "" : s.substr(0, pos);
  bool digits = !tail.empty();
  for (char c : tail)
    digits &= (c >= '0' && c <= '9');
  if (digits) {
    if (!head.empty() && head != "cuda" && head != "gpu" && head != "cuda:gpu")
      return false;
    *out = atoi(tail.c_str());
    return true;
  }
  if (s == "cuda" || s == "gpu" || s == "cuda:gpu") {
    *out = 0;
    return true;
  }
  return false;
}

bool waitDeps(Queue *q, void *events) {
  // In-order stream: events of this queue are already ordered before any new
  // work; events of other queues become stream dependencies.
  if (!events)
    return true;
  for (Event **it = static_cast<Event **>(events); *it; ++it) {
    Event *e = *it;
    if (e->queue == q)
      continue;
    CUDA_TRY(cudaStreamWaitEvent(q->stream, e->ev, 0), return false);
  }
  return true;
}

Event *recordEvent(Queue *q) {
  Event *e = q->getEvent();
  if (!e) {
    nmb::setError("failed to create a CUDA event");
    return nullptr;
  }
  cudaError_t err = cudaEventRecord(e->ev, q->stream);
  if (err != cudaSuccess) {
    nmb::setError("cudaEventRecord failed: %s", cudaGetErrorString(err));
    (void)cudaGetLastError();
    q->returnEvent(e);
    return nullptr;
  }
  return e;
}

// ---------------------------------------------------------------- modules ---
struct Module {
  Queue *queue = nullptr;
  CUmodule cuModule = nullptr; // null for the builtin module
  bool builtin = false;
};

struct Kernel {
  Module *module = nullptr;
  CUfunction func = nullptr;
  int dynSmemBytes = 0;
  int maxThreads = 1024;
  std::string name;
};

// ------------------------------------------------------------------ NVRTC ---
struct NvrtcApi {
  void *handle = nullptr;
  int (*CreateProgram)(void **, const char *, const char *, int,
                       const char *const *, const char *const *) = nullptr;
  int (*CompileProgram)(void *, int, const char *const *) = nullptr;
  int (*GetCUBINSize)(void *, size_t *) = nullptr;
  int (*GetCUBIN)(void *, char *) = nullptr;
  int (*GetProgramLogSize)(void *, size_t *) = nullptr;
  int (*GetProgramLog)(void *, char *) = nullptr;
  int (*DestroyProgram)(void **) = nullptr;
  const char *(*GetErrorString)(int) = nullptr;
  int (*Version)(int *, int *) = nullptr;
  bool ok = false;
};

NvrtcApi &nvrtc() {
  static NvrtcApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    std::vector<std::string> names;
    if (const char *p = getenv("NUMBA_MLIR_NVRTC_PATH"))
      names.push_back(p);
    names.push_back("libnvrtc.so.12");
    names.push_back("/usr/local/cuda/lib64/libnvrtc.so.12");
    names.push_back("libnvrtc.so");
    for (auto &n : names) {
      api.handle = dlopen(n.c_str(), RTLD_NOW | RTLD_LOCAL);
      if (api.handle)
        break;
    }
    if (!api.handle)
      return;
    auto sym = [&](const char *n) { return dlsym(api.handle, n); };
    *(void **)&api.CreateProgram = sym("nvrtcCreateProgram");
    *(void **)&api.CompileProgram = sym("nvrtcCompileProgram");
    *(void **)&api.GetCUBINSize = sym("nvrtcGetCUBINSize");
    *(void **)&api.GetCUBIN = sym("nvrtcGetCUBIN");
    *(void **)&api.GetProgramLogSize = sym("nvrtcGetProgramLogSize");
    *(void **)&api.GetProgramLog = sym("nvrtcGetProgramLog");
    *(void **)&api.DestroyProgram = sym("nvrtcDestroyProgram");
    *(void **)&api.GetErrorString = sym("nvrtcGetErrorString");
    *(void **)&api.Version = sym("nvrtcVersion");
    api.ok = api.CreateProgram && api.CompileProgram && api.GetCUBINSize &&
             api.GetCUBIN && api.GetProgramLogSize && api.GetProgramLog &&
             api.DestroyProgram && api.GetErrorString;
  });
  return api;
}

// The device-side support header handed to every NVRTC compilation under the
// include name "nmb_device.cuh" (generated from kernels/nmb_device.cuh).
const char *const kDeviceHeader =
#include "nmb_device_cuh.inc"
    ;

const char kSourceTag[] = "//NMB200:CUDA-SOURCE";
const char kOptionsTag[] = "//NMB200:OPTIONS";
const char kBuiltinTag[] = "NMB200:BUILTIN";

uint64_t fnv1a(const void *data, size_t n, uint64_t seed) {
  uint64_t h = seed;
  const unsigned char *p = static_cast<const unsigned char *>(data);
  for (size_t i = 0; i < n; ++i) {
    h ^= p[i];
    h *= 1099511628211ull;
  }
  return h;
}

std::string cacheDir() {
  if (const char *p = getenv("NUMBA_MLIR_B200_CACHE_DIR"))
    return p;
  const char *home = getenv("HOME");
  std::string base = home ? home : "/tmp";
  return base + "/.cache/numba_mlir_b200";
}

void mkdirs(const std::string &path) {
  std::string cur;
  for (size_t i = 0; i < path.size(); ++i) {
    cur += path[i];
    if (path[i] == '/' || i + 1 == path.size())
      mkdir(cur.c_str(), 0755);
  }
}

std::mutex gCubinCacheMutex;
std::unordered_map<std::string, std::shared_ptr<std::vector<char>>> gCubinCache;

// CUDA C (tagged blob) -> sm_100a cubin.  In-memory and on-disk caches keyed by
// a hash of source, options and the support header.
std::shared_ptr<std::vector<char>> compileSource(const char *src, size_t size) {
  std::string text(src, size);
  // Options line (optional, second line).
  std::vector<std::string> opts = {"--gpu-architecture=sm_100a", "--std=c++17",
                                   "-default-device"};
  size_t nl = text.find('\n');
  if (nl != std::string::npos) {
    size_t start = nl + 1;
    if (text.compare(start, sizeof(kOptionsTag) - 1, kOptionsTag) == 0) {
      size_t end = text.find('\n', start);
      std::string line = text.substr(start + sizeof(kOptionsTag) - 1,
                                     end == std::string::npos
                                         ? std::string::npos
                                         : end - start - (sizeof(kOptionsTag) - 1));
      size_t i = 0;
      while (i < line.size()) {
        while (i < line.size() && line[i] == ' ')
          ++i;
        size_t j = i;
        while (j < line.size() && line[j] != ' ')
          ++j;
        if (j > i)
          opts.push_back(line.substr(i, j - i));
        i = j;
      }
    }
  }

  uint64_t h1 = fnv1a(text.data(), text.size(), 14695981039346656037ull);
  uint64_t h2 = fnv1a(kDeviceHeader, strlen(kDeviceHeader), h1 ^ 0x9e3779b97f4a7c15ull);
  char key[64];
  snprintf(key, sizeof(key), "%016llx%016llx", (unsigned long long)h1,
           (unsigned long long)h2);
  {
    std::lock_guard<std::mutex> g(gCubinCacheMutex);
    auto it = gCubinCache.find(key);
    if (it != gCubinCache.end())
      return it->second;
  }
  bool useDisk = !envFlag("NUMBA_MLIR_B200_NO_DISK_CACHE");
  std::string path = cacheDir() + "/" + key + ".cubin";
  if (useDisk) {
    if (FILE *f = fopen(path.c_str(), "rb")) {
      auto blob = std::make_shared<std::vector<char>>();
      char buf[65536];
      size_t n;
      while ((n = fread(buf, 1, sizeof(buf), f)) > 0)
        blob->insert(blob->end(), buf, buf + n);
      fclose(f);
      if (blob->size() > 4 && memcmp(blob->data(), "\x7f" "ELF", 4) == 0) {
        std::lock_guard<std::mutex> g(gCubinCacheMutex);
        gCubinCache[key] = blob;
        return blob;
      }
    }
  }

  NvrtcApi &rt = nvrtc();
  if (!rt.ok) {
    nmb::setError("NVRTC (libnvrtc.so.12) could not be loaded; set "
                  "NUMBA_MLIR_NVRTC_PATH");
    return nullptr;
  }
  void *prog = nullptr;
  const char *headerSrc[] = {kDeviceHeader};
  const char *headerNames[] = {"nmb_device.cuh"};
  int rc = rt.CreateProgram(&prog, text.c_str(), "nmb_generated.cu", 1,
                            headerSrc, headerNames);
  if (rc != 0) {
    nmb::setError("nvrtcCreateProgram failed: %s", rt.GetErrorString(rc));
    return nullptr;
  }
  std::vector<const char *> optPtrs;
  for (auto &o : opts)
    optPtrs.push_back(o.c_str());
  rc = rt.CompileProgram(prog, (int)optPtrs.size(), optPtrs.data());
  if (rc != 0) {
    size_t logSize = 0;
    rt.GetProgramLogSize(prog, &logSize);
    std::string log(logSize, '\0');
    if (logSize)
      rt.GetProgramLog(prog, &log[0]);
    if (log.size() > 3500)
      log.resize(3500);
    nmb::setError("NVRTC compilation failed: %s\n%s", rt.GetErrorString(rc),
                  log.c_str());
    rt.DestroyProgram(&prog);
    return nullptr;
  }
  size_t cubinSize = 0;
  rt.GetCUBINSize(prog, &cubinSize);
  auto blob = std::make_shared<std::vector<char>>(cubinSize);
  rt.GetCUBIN(prog, blob->data());
  rt.DestroyProgram(&prog);

  if (useDisk) {
    mkdirs(cacheDir());
    std::string tmp = path + ".tmp" + std::to_string((long)getpid());
    if (FILE *f = fopen(tmp.c_str(), "wb")) {
      fwrite(blob->data(), 1, blob->size(), f);
      fclose(f);
      rename(tmp.c_str(), path.c_str());
    }
  }
  std::lock_guard<std::mutex> g(gCubinCacheMutex);
  gCubinCache[key] = blob;
  return blob;
}

// Blob dump, as NUMBA_MLIR_DUMP_KERNEL_BLOB in GpuRuntime.cpp:37-59.
void dumpBlob(const void *data, size_t size) {
  static bool enabled = envFlag("NUMBA_MLIR_DUMP_KERNEL_BLOB");
  if (!enabled)
    return;
  static std::atomic<int> counter{0};
  char name[128];
  snprintf(name, sizeof(name), "kernel_dump_%d_%d", (int)getpid(), counter++);
  if (FILE *f = fopen(name, "wb")) {
    fwrite(data, 1, size, f);
    fclose(f);
  }
}

uint32_t downPow2(uint32_t x) {
  uint32_t p = 1;
  while (p * 2 <= x && p < 0x80000000u)
    p *= 2;
  return p;
}
uint32_t upPow2(uint32_t x) {
  uint32_t p = 1;
  while (p < x)
    p *= 2;
  return p;
}

bool setDevice(Queue *q) {
  CUDA_TRY(cudaSetDevice(q->device), return false);
  return true;
}

} // namespace

// ------------------------------------------------------- internal helpers ---
namespace nmb {

void registerBuiltin(const char *name, const void *hostFunc, int dynSmemBytes) {
  builtinTable().push_back({name, hostFunc, dynSmemBytes});
}

void setError(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsetError(fmt, ap);
  va_end(ap);
}

bool queueView(void *queue, QueueView *out) {
  if (!queue) {
    setError("invalid (null) queue");
    return false;
  }
  Queue *q = toQueue(queue);
  if (!setDevice(q))
    return false;
  out->stream = q->stream;
  out->device = q->device;
  return true;
}

void *recordEventOn(void *queue) { return recordEvent(toQueue(queue)); }

void noteLaunch() { ++gLaunchCount; }

void *scratchGet(void *queue, size_t bytes) {
  Queue *q = toQueue(queue);
  if (bytes <= q->scratchBytes)
    return q->scratch;
  // Stream-ordered: earlier kernels that use the old region finish before the
  // free takes effect, later ones start after the new allocation.
  if (q->scratch)
    CUDA_TRY(cudaFreeAsync(q->scratch, q->stream), return nullptr);
  q->scratch = nullptr;
  q->scratchBytes = 0;
  size_t want = bytes < (1u << 20) ? (1u << 20) : bytes;
  CUDA_TRY(cudaMallocAsync(&q->scratch, want, q->stream), return nullptr);
  q->scratchBytes = want;
  return q->scratch;
}

uint32_t *statusWord(void *queue) {
  Queue *q = toQueue(queue);
  if (!q->status) {
    void *p = nullptr;
    CUDA_TRY(cudaMallocAsync(&p, 256, q->stream), return nullptr);
    CUDA_TRY(cudaMemsetAsync(p, 0, 256, q->stream), return nullptr);
    q->status = static_cast<uint32_t *>(p);
  }
  return q->status;
}

} // namespace nmb

// ---------------------------------------------------------------- exports ---
GPUX_EXPORT void *gpuxQueueCreate(const char *deviceName) {
  LOG_FUNC();
  int dev = 0;
  if (!parseDeviceIndex(deviceName, &dev)) {
    nmb::setError("unknown device name '%s' (expected cuda:N)",
                  deviceName ? deviceName : "");
    return nullptr;
  }
  int count = 0;
  CUDA_TRY(cudaGetDeviceCount(&count), return nullptr);
  if (dev < 0 || dev >= count) {
    nmb::setError("device index %d out of range (%d CUDA devices)", dev, count);
    return nullptr;
  }
  CUDA_TRY(cudaSetDevice(dev), return nullptr);
  if (!driver().ok) {
    nmb::setError("CUDA driver entry points unavailable");
    return nullptr;
  }
  auto q = new Queue;
  q->device = dev;
  q->deviceName = deviceName ? deviceName : "";
  cudaError_t e = cudaStreamCreateWithFlags(&q->stream, cudaStreamNonBlocking);
  if (e != cudaSuccess) {
    nmb::setError("cudaStreamCreate failed: %s", cudaGetErrorString(e));
    (void)cudaGetLastError();
    q->stream = nullptr;
    delete q;
    return nullptr;
  }
  // Keep freed device memory cached in the stream-ordered pool so repeated
  // result allocations (one per call in generated host code,
  // GpuRuntimeToLlvm.cpp:630-754) do not reach the driver.
  cudaMemPool_t pool;
  if (cudaDeviceGetDefaultMemPool(&pool, dev) == cudaSuccess) {
    uint64_t threshold = UINT64_MAX;
    cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &threshold);
  }
  (void)cudaGetLastError();
  return q;
}

GPUX_EXPORT void gpuxQueueDestroy(void *queue) {
  LOG_FUNC();
  if (!queue)
    return;
  toQueue(queue)->release();
}

GPUX_EXPORT void *gpuxDuplicateQueue(void *nativeStream) {
  LOG_FUNC();
  int dev = 0;
  CUDA_TRY(cudaGetDevice(&dev), return nullptr);
  if (!driver().ok) {
    nmb::setError("CUDA driver entry points unavailable");
    return nullptr;
  }
  auto q = new Queue;
  q->device = dev;
  q->stream = static_cast<cudaStream_t>(nativeStream);
  q->ownsStream = false;
  q->deviceName = "cuda:" + std::to_string(dev);
  return q;
}

GPUX_EXPORT void *gpuxModuleLoad(void *queue, const void *data,
                                 size_t dataSize) {
  LOG_FUNC();
  if (!queue || !data) {
    nmb::setError("gpuxModuleLoad: null queue or blob");
    return nullptr;
  }
  Queue *q = toQueue(queue);
  if (!setDevice(q))
    return nullptr;
  dumpBlob(data, dataSize);
  const char *bytes = static_cast<const char *>(data);

  if (dataSize >= sizeof(kBuiltinTag) - 1 &&
      memcmp(bytes, kBuiltinTag, sizeof(kBuiltinTag) - 1) == 0) {
    auto m = new Module;
    m->queue = q;
    m->builtin = true;
    q->retain();
    return m;
  }

  std::shared_ptr<std::vector<char>> compiled;
  const void *image = data;
  std::string ptxCopy;
  if (dataSize >= sizeof(kSourceTag) - 1 &&
      memcmp(bytes, kSourceTag, sizeof(kSourceTag) - 1) == 0) {
    compiled = compileSource(bytes, dataSize);
    if (!compiled)
      return nullptr;
    image = compiled->data();
  } else if (dataSize >= 4 && memcmp(bytes, "\x7f" "ELF", 4) == 0) {
    // cubin: used as is
  } else if (dataSize >= 4 && (unsigned char)bytes[0] == 0x50 &&
             (unsigned char)bytes[1] == 0xed && (unsigned char)bytes[2] == 0x55 &&
             (unsigned char)bytes[3] == 0xba) {
    // fatbin: used as is
  } else {
    // PTX text must be NUL-terminated for the driver.
    ptxCopy.assign(bytes, dataSize);
    image = ptxCopy.c_str();
  }

  CUmodule cuMod = nullptr;
  char errLog[4096] = {0};
  CUjit_option jitOpts[] = {CU_JIT_ERROR_LOG_BUFFER,
                            CU_JIT_ERROR_LOG_BUFFER_SIZE_BYTES};
  void *jitVals[] = {errLog, (void *)(uintptr_t)sizeof(errLog)};
  CUresult r = DRV(ModuleLoadDataEx, &cuMod, image, 2, jitOpts, jitVals);
  if (r != CUDA_SUCCESS) {
    nmb::setError("cuModuleLoadDataEx failed: %s\n%s", cuErr(r), errLog);
    return nullptr;
  }
  auto m = new Module;
  m->queue = q;
  m->cuModule = cuMod;
  q->retain();
  return m;
}

GPUX_EXPORT void gpuxModuleDestroy(void *module) {
  LOG_FUNC();
  if (!module)
    return;
  Module *m = static_cast<Module *>(module);
  if (m->cuModule) {
    cudaSetDevice(m->queue->device);
    driver().ModuleUnload(m->cuModule);
  }
  m->queue->release();
  delete m;
}

GPUX_EXPORT void *gpuxKernelGet(void *module, const char *name) {
  LOG_FUNC();
  if (!module || !name) {
    nmb::setError("gpuxKernelGet: null module or name");
    return nullptr;
  }
  Module *m = static_cast<Module *>(module);
  if (!setDevice(m->queue))
    return nullptr;
  auto k = std::make_unique<Kernel>();
  k->module = m;
  k->name = name;
  if (m->builtin) {
    const nmb::BuiltinKernel *found = nullptr;
    for (auto &b : builtinTable())
      if (strcmp(b.name, name) == 0)
        found = &b;
    if (!found) {
      nmb::setError("no builtin kernel named '%s'", name);
      return nullptr;
    }
    cudaFunction_t fn = nullptr;
    CUDA_TRY(cudaGetFuncBySymbol(&fn, found->hostFunc), return nullptr);
    k->func = reinterpret_cast<CUfunction>(fn);
    k->dynSmemBytes = found->dynSmemBytes;
  } else {
    CUresult r = DRV(ModuleGetFunction, &k->func, m->cuModule, name);
    if (r != CUDA_SUCCESS) {
      nmb::setError("kernel '%s' not found in module: %s", name, cuErr(r));
      return nullptr;
    }
  }
  int maxThreads = 1024;
  if (driver().FuncGetAttribute(&maxThreads,
                                CU_FUNC_ATTRIBUTE_MAX_THREADS_PER_BLOCK,
                                k->func) == CUDA_SUCCESS)
    k->maxThreads = maxThreads;
  // Allow the full 227 KB of dynamic shared memory.
  int staticSmem = 0;
  driver().FuncGetAttribute(&staticSmem, CU_FUNC_ATTRIBUTE_SHARED_SIZE_BYTES,
                            k->func);
  int optin = 0;
  cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin,
                         m->queue->device);
  if (optin > staticSmem)
    driver().FuncSetAttribute(k->func,
                              CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES,
                              optin - staticSmem);
  return k.release();
}

GPUX_EXPORT void gpuxKernelDestroy(void *kernel) {
  LOG_FUNC();
  delete static_cast<Kernel *>(kernel);
}

namespace {
// The launch itself; false (sticky error set) on failure.
bool launchKernel(void *queue, void *kernel, size_t gridX, size_t gridY, size_t gridZ, size_t blockX,
                  size_t blockY, size_t blockZ, void *events, void *params);
} // namespace

GPUX_EXPORT void *gpuxLaunchKernel(void *queue, void *kernel, size_t gridX,
                                   size_t gridY, size_t gridZ, size_t blockX,
                                   size_t blockY, size_t blockZ, void *events,
                                   void *params) {
  LOG_FUNC();
  if (!launchKernel(queue, kernel, gridX, gridY, gridZ, blockX, blockY, blockZ, events, params))
    return nullptr;
  return recordEvent(toQueue(queue));
}

// gpuxLaunchKernel for callers that order their work by the queue alone and
// would destroy the returned event at once: no event is recorded.  Returns 1,
// or 0 with the sticky error set.
GPUX_EXPORT int gpuxLaunchKernelNoEvent(void *queue, void *kernel, size_t gridX, size_t gridY, size_t gridZ,
                                        size_t blockX, size_t blockY, size_t blockZ, void *events,
                                        void *params) {
  LOG_FUNC();
  return launchKernel(queue, kernel, gridX, gridY, gridZ, blockX, blockY, blockZ, events, params) ? 1 : 0;
}

namespace {
bool launchKernel(void *queue, void *kernel, size_t gridX, size_t gridY, size_t gridZ, size_t blockX,
                  size_t blockY, size_t blockZ, void *events, void *params) {
  if (!queue || !kernel) {
    nmb::setError("gpuxLaunchKernel: null queue or kernel");
    return false;
  }
  Queue *q = toQueue(queue);
  Kernel *k = static_cast<Kernel *>(kernel);
  if (!setDevice(q) || !waitDeps(q, events))
    return false;

  // Argument marshalling (Queue::setKernelArg, GpuRuntime.cpp:302-351).
  static const int kTypeSize[] = {0, 1, 1, 2, 4, 8, 4, 8, 8};
  void *args[256];
  uint64_t localOffsets[64];
  size_t nargs = 0, nlocal = 0;
  size_t dynSmem = (size_t)k->dynSmemBytes;
  if (params) {
    for (GPUXParamDesc *p = static_cast<GPUXParamDesc *>(params);
         !(p->data == nullptr && p->size == 0 && p->type == GPUX_PARAM_NULL);
         ++p) {
      if (nargs >= 256) {
        nmb::setError("gpuxLaunchKernel: more than 256 parameters");
        return false;
      }
      if (p->type <= GPUX_PARAM_NULL || p->type > GPUX_PARAM_PTR) {
        nmb::setError("Unhandled param type: %d", (int)p->type);
        return false;
      }
      if (p->type == GPUX_PARAM_PTR && p->data == nullptr) {
        if (nlocal >= 64) {
          nmb::setError("gpuxLaunchKernel: more than 64 local-memory params");
          return false;
        }
        dynSmem = (dynSmem + 15) & ~size_t(15);
        localOffsets[nlocal] = dynSmem;
        dynSmem += (size_t)p->size;
        args[nargs++] = &localOffsets[nlocal++];
        continue;
      }
      if (p->size != kTypeSize[p->type]) {
        nmb::setError("param %zu: size %d does not match type %d", nargs,
                      (int)p->size, (int)p->type);
        return false;
      }
      args[nargs++] = const_cast<void *>(p->data);
    }
  }

  if (gridX && gridY && gridZ && blockX && blockY && blockZ) {
    if (gridX > 0x7fffffffull || gridY > 65535 || gridZ > 65535) {
      nmb::setError("grid (%zu,%zu,%zu) exceeds CUDA limits (2^31-1,65535,65535)",
                    gridX, gridY, gridZ);
      return false;
    }
    CU_TRY(DRV(LaunchKernel, k->func, (unsigned)gridX, (unsigned)gridY,
                                 (unsigned)gridZ, (unsigned)blockX,
                                 (unsigned)blockY, (unsigned)blockZ,
                                 (unsigned)dynSmem, (CUstream)q->stream, args,
                                 nullptr),
           return false);
    ++gLaunchCount;
  }
  return true;
}
} // namespace

// Host-side bound on gpuxWait: NUMBA_MLIR_GPU_WAIT_TIMEOUT_MS (read at every
// call, 0 or unset = wait for as long as it takes, like the reference's
// event.wait(), GpuRuntime.cpp:395-404).  With a bound the event is polled;
// when the time runs out the call returns with the sticky error set and the
// device work is left running.
GPUX_EXPORT void gpuxWait(void *queue, void *event) {
  LOG_FUNC();
  (void)queue;
  if (!event)
    return;
  Event *e = static_cast<Event *>(event);
  const char *limit = getenv("NUMBA_MLIR_GPU_WAIT_TIMEOUT_MS");
  const long ms = limit && *limit ? strtol(limit, nullptr, 10) : 0;
  if (ms <= 0) {
    CUDA_TRY(cudaEventSynchronize(e->ev), return);
    return;
  }
  timespec t0;
  clock_gettime(CLOCK_MONOTONIC, &t0);
  for (unsigned spins = 0;; ++spins) {
    cudaError_t st = cudaEventQuery(e->ev);
    if (st == cudaSuccess)
      return;
    if (st != cudaErrorNotReady) {
      nmb::setError("gpuxWait: cudaEventQuery failed: %s", cudaGetErrorString(st));
      (void)cudaGetLastError();
      return;
    }
    (void)cudaGetLastError();
    timespec t1;
    clock_gettime(CLOCK_MONOTONIC, &t1);
    const double waited = (t1.tv_sec - t0.tv_sec) * 1e3 + (t1.tv_nsec - t0.tv_nsec) * 1e-6;
    if (waited > (double)ms) {
      nmb::setError("gpuxWait: the event was not reached within %ld ms "
                    "(NUMBA_MLIR_GPU_WAIT_TIMEOUT_MS); the device work is still in flight",
                    ms);
      return;
    }
    if (spins > 1000)
      usleep(50); // the first polls are back to back: short waits stay short
  }
}

GPUX_EXPORT void gpuxDestroyEvent(void *queue, void *event) {
  LOG_FUNC();
  (void)queue;
  if (!event)
    return;
  Event *e = static_cast<Event *>(event);
  e->queue->returnEvent(e);
}

GPUX_EXPORT void gpuxAlloc(void *queue, size_t size, size_t alignment, int type,
                           void *events, GPUXAllocResult *ret) {
  LOG_FUNC();
  if (ret)
    *ret = {nullptr, nullptr};
  if (!queue || !ret) {
    nmb::setError("gpuxAlloc: null queue or result");
    return;
  }
  Queue *q = toQueue(queue);
  if (!setDevice(q) || !waitDeps(q, events))
    return;
  if (alignment > 256) {
    nmb::setError("gpuxAlloc: alignment %zu above the 256 bytes CUDA gives",
                  alignment);
    return;
  }
  void *mem = nullptr;
  size_t bytes = size ? size : 1;
  switch (type) {
  case GPUX_ALLOC_DEVICE:
    // Stream-ordered: usable by later work on this queue without a host wait.
    CUDA_TRY(cudaMallocAsync(&mem, bytes, q->stream), {
      nmb::setError("Failed to allocate device memory (%zu bytes)", size);
      return;
    });
    break;
  case GPUX_ALLOC_SHARED:
    CUDA_TRY(cudaMallocManaged(&mem, bytes), {
      nmb::setError("Failed to allocate shared memory (%zu bytes)", size);
      return;
    });
    break;
  case GPUX_ALLOC_HOST:
    CUDA_TRY(cudaMallocHost(&mem, bytes), {
      nmb::setError("Failed to allocate host memory (%zu bytes)", size);
      return;
    });
    break;
  case GPUX_ALLOC_LOCAL:
    // Work-group-local buffers have no host-side pointer; their size travels
    // in the launch parameter (GpuRuntime.cpp:239-241).
    break;
  default:
    nmb::setError("Invalid allocation type %d", type);
    return;
  }
  if (mem) {
    std::lock_guard<std::mutex> g(q->mutex);
    q->allocs[mem] = type;
  }
  // Buffers keep the queue alive (GpuRuntime.cpp:248-250).
  q->retain();
  ret->ptr = mem;
  ret->event = recordEvent(q);
}

GPUX_EXPORT void gpuxDeAlloc(void *queue, void *ptr) {
  LOG_FUNC();
  if (!queue)
    return;
  Queue *q = toQueue(queue);
  if (ptr) {
    int type = -1;
    {
      std::lock_guard<std::mutex> g(q->mutex);
      auto it = q->allocs.find(ptr);
      if (it != q->allocs.end()) {
        type = it->second;
        q->allocs.erase(it);
      }
    }
    cudaSetDevice(q->device);
    if (type == GPUX_ALLOC_DEVICE)
      cudaFreeAsync(ptr, q->stream);
    else if (type == GPUX_ALLOC_SHARED)
      cudaFree(ptr);
    else if (type == GPUX_ALLOC_HOST)
      cudaFreeHost(ptr);
    else {
      // not a buffer of this queue (or freed before): it holds no reference
      nmb::setError("gpuxDeAlloc: pointer %p was not allocated by this queue",
                    ptr);
      return;
    }
    (void)cudaGetLastError();
  }
  q->release();
}

GPUX_EXPORT void gpuxSuggestBlockSize(void *queue, void *kernel,
                                      const uint32_t *gridSize,
                                      uint32_t *blockSize, size_t numDims) {
  LOG_FUNC();
  if (!kernel || !gridSize || !blockSize || numDims < 1 || numDims > 3) {
    nmb::setError("gpuxSuggestBlockSize: invalid arguments");
    return;
  }
  Kernel *k = static_cast<Kernel *>(kernel);
  if (queue)
    cudaSetDevice(toQueue(queue)->device);
  int minGrid = 0, best = 0;
  if (driver().OccupancyMaxPotentialBlockSize(&minGrid, &best, k->func, nullptr,
                                              (size_t)k->dynSmemBytes,
                                              0) != CUDA_SUCCESS ||
      best <= 0)
    best = k->maxThreads;
  // Generated one-element-per-work-item kernels gain nothing beyond 256.
  if (best > 256)
    best = 256;
  uint32_t maxWg = downPow2((uint32_t)best);
  static const uint32_t kDimLimit[3] = {1024, 1024, 64};
  for (size_t i = 0; i < numDims; ++i) {
    uint32_t g = gridSize[i];
    if (g > 1) {
      uint32_t l = g < maxWg ? g : maxWg;
      if (l > kDimLimit[i])
        l = kDimLimit[i];
      blockSize[i] = l;
      maxWg /= upPow2(l);
      if (maxWg == 0)
        maxWg = 1;
    } else {
      blockSize[i] = 1;
    }
  }
}

// ------------------------------------------------------------- extensions ---
GPUX_EXPORT void *gpuxMemcpy(void *queue, void *dst, const void *src,
                             size_t bytes, int kind, void *events) {
  LOG_FUNC();
  if (!queue) {
    nmb::setError("gpuxMemcpy: null queue");
    return nullptr;
  }
  Queue *q = toQueue(queue);
  if (!setDevice(q) || !waitDeps(q, events))
    return nullptr;
  cudaMemcpyKind k = cudaMemcpyDefault;
  if (kind == GPUX_COPY_H2D)
    k = cudaMemcpyHostToDevice;
  else if (kind == GPUX_COPY_D2H)
    k = cudaMemcpyDeviceToHost;
  else if (kind == GPUX_COPY_D2D)
    k = cudaMemcpyDeviceToDevice;
  if (bytes)
    CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, k, q->stream), return nullptr);
  return recordEvent(q);
}

GPUX_EXPORT void *gpuxMemset(void *queue, void *dst, int value, size_t bytes,
                             void *events) {
  LOG_FUNC();
  if (!queue) {
    nmb::setError("gpuxMemset: null queue");
    return nullptr;
  }
  Queue *q = toQueue(queue);
  if (!setDevice(q) || !waitDeps(q, events))
    return nullptr;
  if (bytes)
    CUDA_TRY(cudaMemsetAsync(dst, value, bytes, q->stream), return nullptr);
  return recordEvent(q);
}

GPUX_EXPORT int gpuxQueueWaitEvents(void *queue, void *events) {
  LOG_FUNC();
  if (!queue) {
    nmb::setError("gpuxQueueWaitEvents: null queue");
    return 1;
  }
  Queue *q = toQueue(queue);
  return setDevice(q) && waitDeps(q, events) ? 0 : 1;
}

GPUX_EXPORT int gpuxQueueWaitStream(void *queue, void *nativeStream) {
  LOG_FUNC();
  if (!queue) {
    nmb::setError("gpuxQueueWaitStream: null queue");
    return 1;
  }
  Queue *q = toQueue(queue);
  cudaStream_t other = static_cast<cudaStream_t>(nativeStream);
  if (other == q->stream)
    return 0;
  if (!setDevice(q))
    return 1;
  Event *e = q->getEvent();
  if (!e) {
    nmb::setError("failed to create a CUDA event");
    return 1;
  }
  bool ok = true;
  CUDA_TRY(cudaEventRecord(e->ev, other), ok = false);
  if (ok)
    CUDA_TRY(cudaStreamWaitEvent(q->stream, e->ev, 0), ok = false);
  q->returnEvent(e);
  return ok ? 0 : 1;
}

// ------------------------------------------------------------ peer memory ---
GPUX_EXPORT void *gpuxPeerAlloc(void *queue, size_t size) {
  LOG_FUNC();
  if (!queue || !size) {
    nmb::setError("gpuxPeerAlloc: null queue or zero size");
    return nullptr;
  }
  Queue *q = toQueue(queue);
  if (!setDevice(q))
    return nullptr;
  void *p = nullptr;
  // plain cudaMalloc: memory of a stream-ordered pool cannot be exported
  CUDA_TRY(cudaMalloc(&p, size), return nullptr);
  CUDA_TRY(cudaMemset(p, 0, size), cudaFree(p); return nullptr);
  CUDA_TRY(cudaDeviceSynchronize(), cudaFree(p); return nullptr);
  return p;
}

GPUX_EXPORT void gpuxPeerFree(void *queue, void *ptr) {
  LOG_FUNC();
  if (!queue || !ptr)
    return;
  if (!setDevice(toQueue(queue)))
    return;
  CUDA_TRY(cudaFree(ptr), return);
}

GPUX_EXPORT int gpuxPeerExport(void *ptr, void *handle) {
  LOG_FUNC();
  static_assert(sizeof(cudaIpcMemHandle_t) == GPUX_PEER_HANDLE_BYTES, "handle size");
  if (!ptr || !handle) {
    nmb::setError("gpuxPeerExport: null argument");
    return 1;
  }
  cudaIpcMemHandle_t h;
  CUDA_TRY(cudaIpcGetMemHandle(&h, ptr), return 1);
  memcpy(handle, &h, sizeof(h));
  return 0;
}

GPUX_EXPORT void *gpuxPeerOpen(void *queue, const void *handle) {
  LOG_FUNC();
  if (!queue || !handle) {
    nmb::setError("gpuxPeerOpen: null argument");
    return nullptr;
  }
  if (!setDevice(toQueue(queue)))
    return nullptr;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void *p = nullptr;
  CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), return nullptr);
  return p;
}

GPUX_EXPORT void gpuxPeerClose(void *queue, void *ptr) {
  LOG_FUNC();
  if (!queue || !ptr)
    return;
  if (!setDevice(toQueue(queue)))
    return;
  CUDA_TRY(cudaIpcCloseMemHandle(ptr), return);
}

GPUX_EXPORT void *gpuxRecordEvent(void *queue) {
  LOG_FUNC();
  if (!queue) {
    nmb::setError("gpuxRecordEvent: null queue");
    return nullptr;
  }
  Queue *q = toQueue(queue);
  if (!setDevice(q))
    return nullptr;
  return recordEvent(q);
}

GPUX_EXPORT float gpuxEventElapsedMs(void *startEvent, void *endEvent) {
  LOG_FUNC();
  if (!startEvent || !endEvent) {
    nmb::setError("gpuxEventElapsedMs: null event");
    return -1.f;
  }
  float ms = -1.f;
  CUDA_TRY(cudaEventElapsedTime(&ms, static_cast<Event *>(startEvent)->ev,
                                static_cast<Event *>(endEvent)->ev),
           return -1.f);
  return ms;
}

GPUX_EXPORT void gpuxQueueSynchronize(void *queue) {
  LOG_FUNC();
  if (!queue)
    return;
  Queue *q = toQueue(queue);
  if (!setDevice(q))
    return;
  CUDA_TRY(cudaStreamSynchronize(q->stream), return);
}

GPUX_EXPORT void *gpuxQueueGetStream(void *queue) {
  return queue ? (void *)toQueue(queue)->stream : nullptr;
}

GPUX_EXPORT int gpuxQueueGetDevice(void *queue) {
  return queue ? toQueue(queue)->device : -1;
}

// Number of multiprocessors of the queue's device (launch shapes are sized in
// multiples of it); -1 on error.
GPUX_EXPORT int gpuxQueueGetSmCount(void *queue) {
  if (!queue) {
    nmb::setError("gpuxQueueGetSmCount: null queue");
    return -1;
  }
  int n = 0;
  CUDA_TRY(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, toQueue(queue)->device), return -1);
  return n;
}

// Test hook for host-side failure injection: the next `count` calls of the
// driver entry point `name` ("cuLaunchKernel", "cuModuleLoadDataEx",
// "cuModuleGetFunction") made by this library return `code` (a CUresult)
// without reaching the driver; count 0 clears a pending injection.  Nothing on
// the device is made to fail.
GPUX_EXPORT void gpuxTestInjectDriverFault(const char *name, int code, int count) {
  std::lock_guard<std::mutex> g(gDriverFault.mutex);
  gDriverFault.name = name ? name : "";
  gDriverFault.code = code;
  gDriverFault.remaining = name && count > 0 ? count : 0;
}

// Device address of the queue's status word: 0 while every bounded device-side
// wait succeeded; a kernel that gave up waiting stores a non-zero code.
GPUX_EXPORT void *gpuxQueueStatusPtr(void *queue) {
  LOG_FUNC();
  if (!queue) {
    nmb::setError("gpuxQueueStatusPtr: null queue");
    return nullptr;
  }
  if (!setDevice(toQueue(queue)))
    return nullptr;
  return nmb::statusWord(queue);
}

GPUX_EXPORT const char *gpuxGetLastError(void) {
  std::lock_guard<std::mutex> g(gErrMutex);
  return gHasError ? gLastError.c_str() : nullptr;
}

GPUX_EXPORT void gpuxClearLastError(void) {
  std::lock_guard<std::mutex> g(gErrMutex);
  gHasError = false;
}

GPUX_EXPORT uint64_t gpuxLaunchCount(void) { return gLaunchCount.load(); }

// CUDA graphs: record the launches submitted to a queue, then replay them with
// one call (removes the per-launch host cost of short kernels).
struct Graph {
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  int device = 0;
};

GPUX_EXPORT void gpuxGraphBegin(void *queue) {
  LOG_FUNC();
  if (!queue) {
    nmb::setError("gpuxGraphBegin: null queue");
    return;
  }
  Queue *q = toQueue(queue);
  if (!setDevice(q))
    return;
  CUDA_TRY(cudaStreamBeginCapture(q->stream, cudaStreamCaptureModeThreadLocal), return);
}

GPUX_EXPORT void *gpuxGraphEnd(void *queue) {
  LOG_FUNC();
  if (!queue) {
    nmb::setError("gpuxGraphEnd: null queue");
    return nullptr;
  }
  Queue *q = toQueue(queue);
  if (!setDevice(q))
    return nullptr;
  auto g = std::make_unique<Graph>();
  g->device = q->device;
  CUDA_TRY(cudaStreamEndCapture(q->stream, &g->graph), return nullptr);
  CUDA_TRY(cudaGraphInstantiate(&g->exec, g->graph, 0), {
    cudaGraphDestroy(g->graph);
    return nullptr;
  });
  return g.release();
}

GPUX_EXPORT void *gpuxGraphLaunch(void *queue, void *graph) {
  LOG_FUNC();
  if (!queue || !graph) {
    nmb::setError("gpuxGraphLaunch: null queue or graph");
    return nullptr;
  }
  Queue *q = toQueue(queue);
  if (!setDevice(q))
    return nullptr;
  CUDA_TRY(cudaGraphLaunch(static_cast<Graph *>(graph)->exec, q->stream), return nullptr);
  return recordEvent(q);
}

GPUX_EXPORT void gpuxGraphDestroy(void *graph) {
  LOG_FUNC();
  if (!graph)
    return;
  Graph *g = static_cast<Graph *>(graph);
  cudaSetDevice(g->device);
  if (g->exec)
    cudaGraphExecDestroy(g->exec);
  if (g->graph)
    cudaGraphDestroy(g->graph);
  (void)cudaGetLastError();
  delete g;
}

// Host-only helper: compiles a tagged CUDA C blob to an sm_100a cubin without
// touching a device.  The result is malloc()ed; release with gpuxFreeHostBlob.
GPUX_EXPORT void *gpuxCompileToCubin(const void *data, size_t dataSize,
                                     size_t *outSize) {
  LOG_FUNC();
  if (!data || !outSize) {
    nmb::setError("gpuxCompileToCubin: null argument");
    return nullptr;
  }
  auto blob = compileSource(static_cast<const char *>(data), dataSize);
  if (!blob)
    return nullptr;
  void *out = malloc(blob->size());
  memcpy(out, blob->data(), blob->size());
  *outSize = blob->size();
  return out;
}

GPUX_EXPORT void gpuxFreeHostBlob(void *blob) { free(blob); }

// Names of the builtin kernels, '\n'-separated (for tests and tooling).
GPUX_EXPORT const char *gpuxBuiltinKernelNames(void) {
  static std::string names;
  static std::once_flag once;
  std::call_once(once, [] {
    for (auto &b : builtinTable()) {
      names += b.name;
      names += '\n';
    }
  });
  return names.c_str();
}
