// Native launch path of the Python front end (CPython extension `_fastcall`).
//
// Counterpart of the reference's native unboxing and dispatch
// (numba_mlir/numba_mlir/python_runtime/lib/Boxing.cpp:45-136 turns array
// arguments into memref descriptors in C++; the generated host function then
// builds the GPUParamDesc array and calls gpuxLaunchKernel,
// mlir/lib/Conversion/GpuRuntimeToLlvm.cpp:444-628).  The hot part of a call --
// reading pointers and shapes out of the argument objects, building the
// GPUParamDesc array, gpuxLaunchKernel, gpuxDestroyEvent -- runs here instead
// of in Python/ctypes:
//
//   init(launch, destroy_event)            addresses of the two C-ABI entry points
//   launch_kernel(queue, kernel, grid, block, layout, args, tail)
//                                          one @kernel launch from its Python arguments
//   replay(queue, launches, args)          the launches of a recorded njit plan
//   signature(args)                        the plan-cache key of a call's arguments
//
// Nothing here touches the device; a failed launch (NULL event) is reported as
// RuntimeError and the Python side reads the runtime's message.

#define PY_SSIZE_T_CLEAN
#include <Python.h>

#include <chrono>
#include <cstdint>
#include <cstring>

namespace {

struct GPUParamDesc {
  const void *data;
  int32_t size;
  int32_t type;
};
enum { P_NULL = 0, P_BOOL, P_INT8, P_INT16, P_INT32, P_INT64, P_FLOAT32, P_FLOAT64, P_PTR };

typedef void *(*LaunchFn)(void *, void *, size_t, size_t, size_t, size_t, size_t, size_t, void *, void *);
typedef void (*DestroyEventFn)(void *, void *);

typedef int (*LaunchNoEventFn)(void *, void *, size_t, size_t, size_t, size_t, size_t, size_t, void *, void *);
LaunchFn gLaunch = nullptr;
LaunchNoEventFn gLaunchNoEvent = nullptr; // preferred when set: nothing to destroy
DestroyEventFn gDestroyEvent = nullptr;
PyObject *sAddr = nullptr, *sShape = nullptr, *sStrides = nullptr, *sItemsize = nullptr, *sTraceSig = nullptr,
         *sExtent = nullptr, *sAlias = nullptr;

constexpr int kMaxParams = 256;

union Slot {
  void *p;
  int64_t i64;
  int32_t i32;
  int16_t i16;
  int8_t i8;
  float f32;
  double f64;
  bool b;
};

struct Params {
  GPUParamDesc desc[kMaxParams + 1];
  Slot slot[kMaxParams];
  int n = 0;

  bool room() {
    if (n >= kMaxParams) {
      PyErr_SetString(PyExc_ValueError, "too many kernel parameters");
      return false;
    }
    return true;
  }
  bool ptr(uint64_t v) {
    if (!room())
      return false;
    slot[n].p = reinterpret_cast<void *>(v);
    desc[n] = {&slot[n], 8, P_PTR};
    ++n;
    return true;
  }
  bool i64(int64_t v) {
    if (!room())
      return false;
    slot[n].i64 = v;
    desc[n] = {&slot[n], 8, P_INT64};
    ++n;
    return true;
  }
  bool local(int64_t bytes) {
    if (!room())
      return false;
    desc[n] = {nullptr, (int32_t)bytes, P_PTR};
    ++n;
    return true;
  }
  // code: one of the scalar kind letters below
  bool scalar(char code, PyObject *v) {
    if (!room())
      return false;
    Slot &s = slot[n];
    switch (code) {
    case 'q':
    case 'Q': {
      s.i64 = code == 'q' ? PyLong_AsLongLong(v) : (int64_t)PyLong_AsUnsignedLongLongMask(v);
      desc[n] = {&s, 8, P_INT64};
      break;
    }
    case 'i':
    case 'I':
      s.i32 = (int32_t)PyLong_AsLongLong(v);
      desc[n] = {&s, 4, P_INT32};
      break;
    case 'h':
    case 'H':
      s.i16 = (int16_t)PyLong_AsLongLong(v);
      desc[n] = {&s, 2, P_INT16};
      break;
    case 'c':
    case 'C':
      s.i8 = (int8_t)PyLong_AsLongLong(v);
      desc[n] = {&s, 1, P_INT8};
      break;
    case 'f':
      s.f32 = (float)PyFloat_AsDouble(v);
      desc[n] = {&s, 4, P_FLOAT32};
      break;
    case 'd':
      s.f64 = PyFloat_AsDouble(v);
      desc[n] = {&s, 8, P_FLOAT64};
      break;
    case 'b':
      s.b = PyObject_IsTrue(v) == 1;
      desc[n] = {&s, 1, P_BOOL};
      break;
    default:
      PyErr_Format(PyExc_ValueError, "unknown parameter code '%c'", code);
      return false;
    }
    if (PyErr_Occurred())
      return false;
    ++n;
    return true;
  }
  void finish() { desc[n] = {nullptr, 0, P_NULL}; }
};

bool dims3(PyObject *t, size_t out[3]) {
  out[0] = out[1] = out[2] = 1;
  if (!PyTuple_Check(t) || PyTuple_GET_SIZE(t) < 1 || PyTuple_GET_SIZE(t) > 3) {
    PyErr_SetString(PyExc_ValueError, "grid and block are tuples of 1 to 3 integers");
    return false;
  }
  for (Py_ssize_t i = 0; i < PyTuple_GET_SIZE(t); ++i) {
    out[i] = (size_t)PyLong_AsUnsignedLongLong(PyTuple_GET_ITEM(t, i));
    if (PyErr_Occurred())
      return false;
  }
  return true;
}

bool do_launch(void *queue, void *kernel, const size_t g[3], const size_t b[3], Params &p) {
  if (gLaunchNoEvent) {
    p.finish();
    if (!gLaunchNoEvent(queue, kernel, g[0], g[1], g[2], b[0], b[1], b[2], nullptr, p.desc)) {
      PyErr_SetString(PyExc_RuntimeError, "gpuxLaunchKernelNoEvent failed");
      return false;
    }
    return true;
  }
  if (!gLaunch || !gDestroyEvent) {
    PyErr_SetString(PyExc_RuntimeError, "_fastcall.init was not called");
    return false;
  }
  p.finish();
  void *ev = gLaunch(queue, kernel, g[0], g[1], g[2], b[0], b[1], b[2], nullptr, p.desc);
  if (!ev) {
    PyErr_SetString(PyExc_RuntimeError, "gpuxLaunchKernel returned NULL");
    return false;
  }
  gDestroyEvent(queue, ev);
  return true;
}

// Device address of an array argument (attribute `_addr`, set when the array is built).
bool array_addr(PyObject *a, uint64_t *out) {
  PyObject *v = PyObject_GetAttr(a, sAddr);
  if (!v)
    return false;
  *out = PyLong_AsUnsignedLongLong(v);
  Py_DECREF(v);
  return !PyErr_Occurred();
}

PyObject *py_init(PyObject *, PyObject *args) {
  unsigned long long launch = 0, destroy = 0, launch_no_event = 0;
  if (!PyArg_ParseTuple(args, "KK|K", &launch, &destroy, &launch_no_event))
    return nullptr;
  gLaunch = reinterpret_cast<LaunchFn>(launch);
  gDestroyEvent = reinterpret_cast<DestroyEventFn>(destroy);
  gLaunchNoEvent = reinterpret_cast<LaunchNoEventFn>(launch_no_event);
  Py_RETURN_NONE;
}

// launch_kernel(queue, kernel, grid, block, layout, args, tail)
// layout: one entry per Python argument -- bytes "A<ndim><C|S>" is written as the
// three characters 'A', chr(ndim), 'C' or 'S' (strided: element strides follow
// the shape), or one scalar code letter; tail: tuple of int64 values appended
// (the global sizes), optionally followed by a negative number -(local bytes).
// With `repeat` > 0 the launch is issued that many times in a row and the host
// seconds per launch are returned.
PyObject *py_launch_kernel(PyObject *, PyObject *pyargs) {
  unsigned long long queue, kernel;
  PyObject *grid, *block, *args, *tail;
  const char *layout;
  Py_ssize_t layout_len;
  Py_ssize_t repeat = 0;
  if (!PyArg_ParseTuple(pyargs, "KKOOy#OO|n", &queue, &kernel, &grid, &block, &layout, &layout_len, &args, &tail,
                        &repeat))
    return nullptr;
  size_t g[3], b[3];
  if (!dims3(grid, g) || !dims3(block, b))
    return nullptr;
  if (!PyTuple_Check(args) || !PyTuple_Check(tail)) {
    PyErr_SetString(PyExc_TypeError, "args and tail must be tuples");
    return nullptr;
  }
  Params p;
  Py_ssize_t ai = 0;
  for (Py_ssize_t k = 0; k < layout_len; ++ai) {
    if (ai >= PyTuple_GET_SIZE(args)) {
      PyErr_SetString(PyExc_ValueError, "fewer arguments than the kernel takes");
      return nullptr;
    }
    PyObject *a = PyTuple_GET_ITEM(args, ai);
    if (layout[k] == 'A') {
      const int ndim = (unsigned char)layout[k + 1];
      const bool strided = layout[k + 2] == 'S';
      k += 3;
      uint64_t addr;
      if (!array_addr(a, &addr) || !p.ptr(addr))
        return nullptr;
      PyObject *shape = PyObject_GetAttr(a, sShape);
      if (!shape)
        return nullptr;
      bool ok = PyTuple_Check(shape) && PyTuple_GET_SIZE(shape) == ndim;
      for (int d = 0; ok && d < ndim; ++d)
        ok = p.i64(PyLong_AsLongLong(PyTuple_GET_ITEM(shape, d))) && !PyErr_Occurred();
      Py_DECREF(shape);
      if (!ok) {
        if (!PyErr_Occurred())
          PyErr_SetString(PyExc_ValueError, "array rank differs from the compiled kernel's");
        return nullptr;
      }
      if (strided) {
        PyObject *strides = PyObject_GetAttr(a, sStrides);
        PyObject *item = strides ? PyObject_GetAttr(a, sItemsize) : nullptr;
        if (!item) {
          Py_XDECREF(strides);
          return nullptr;
        }
        const long long it = PyLong_AsLongLong(item);
        ok = it > 0 && PyTuple_Check(strides) && PyTuple_GET_SIZE(strides) == ndim;
        for (int d = 0; ok && d < ndim; ++d) {
          const long long st = PyLong_AsLongLong(PyTuple_GET_ITEM(strides, d));
          // Python's floor division: strides may be negative
          long long q = st / it;
          if ((st % it != 0) && ((st < 0) != (it < 0)))
            --q;
          ok = p.i64(q) && !PyErr_Occurred();
        }
        Py_DECREF(strides);
        Py_DECREF(item);
        if (!ok) {
          if (!PyErr_Occurred())
            PyErr_SetString(PyExc_ValueError, "bad strides");
          return nullptr;
        }
      }
    } else {
      if (!p.scalar(layout[k], a))
        return nullptr;
      ++k;
    }
  }
  for (Py_ssize_t t = 0; t < PyTuple_GET_SIZE(tail); ++t) {
    const long long v = PyLong_AsLongLong(PyTuple_GET_ITEM(tail, t));
    if (PyErr_Occurred())
      return nullptr;
    if (v < 0 ? !p.local(-v) : !p.i64(v))
      return nullptr;
  }
  if (repeat > 0) {
    // the same launch `repeat` times without returning to the interpreter:
    // what the runtime and the driver cost per launch, in seconds
    const auto t0 = std::chrono::steady_clock::now();
    for (Py_ssize_t r = 0; r < repeat; ++r)
      if (!do_launch(reinterpret_cast<void *>(queue), reinterpret_cast<void *>(kernel), g, b, p))
        return nullptr;
    const std::chrono::duration<double> dt = std::chrono::steady_clock::now() - t0;
    return PyFloat_FromDouble(dt.count() / (double)repeat);
  }
  if (!do_launch(reinterpret_cast<void *>(queue), reinterpret_cast<void *>(kernel), g, b, p))
    return nullptr;
  Py_RETURN_NONE;
}

// replay(queue, launches, args): launches is a tuple of
// (kernel, grid, block, codes, sources); codes has one letter per parameter:
// 'p' = device address of args[sources[k]], a scalar letter = args[sources[k]]
// converted, 'k' = the int64 constant sources[k].
PyObject *py_replay(PyObject *, PyObject *pyargs) {
  unsigned long long queue;
  PyObject *launches, *args;
  if (!PyArg_ParseTuple(pyargs, "KOO", &queue, &launches, &args))
    return nullptr;
  if (!PyTuple_Check(launches) || !PyTuple_Check(args)) {
    PyErr_SetString(PyExc_TypeError, "launches and args must be tuples");
    return nullptr;
  }
  const Py_ssize_t nargs = PyTuple_GET_SIZE(args);
  for (Py_ssize_t l = 0; l < PyTuple_GET_SIZE(launches); ++l) {
    unsigned long long kernel;
    PyObject *grid, *block, *sources;
    const char *codes;
    Py_ssize_t ncodes;
    if (!PyArg_ParseTuple(PyTuple_GET_ITEM(launches, l), "KOOy#O", &kernel, &grid, &block, &codes, &ncodes,
                          &sources))
      return nullptr;
    size_t g[3], b[3];
    if (!dims3(grid, g) || !dims3(block, b))
      return nullptr;
    if (!PyTuple_Check(sources) || PyTuple_GET_SIZE(sources) != ncodes) {
      PyErr_SetString(PyExc_ValueError, "one source per parameter code");
      return nullptr;
    }
    Params p;
    for (Py_ssize_t k = 0; k < ncodes; ++k) {
      PyObject *src = PyTuple_GET_ITEM(sources, k);
      const long long v = PyLong_AsLongLong(src);
      if (PyErr_Occurred())
        return nullptr;
      if (codes[k] == 'k') {
        if (!p.i64(v))
          return nullptr;
        continue;
      }
      if (v < 0 || v >= nargs) {
        PyErr_SetString(PyExc_IndexError, "plan refers to an argument the call does not have");
        return nullptr;
      }
      PyObject *a = PyTuple_GET_ITEM(args, v);
      if (codes[k] == 'p') {
        uint64_t addr;
        if (!array_addr(a, &addr) || !p.ptr(addr))
          return nullptr;
      } else if (!p.scalar(codes[k], a)) {
        return nullptr;
      }
    }
    if (!do_launch(reinterpret_cast<void *>(queue), reinterpret_cast<void *>(kernel), g, b, p))
      return nullptr;
  }
  Py_RETURN_NONE;
}

// signature(args, array_type): the plan-cache key of a call -- per array its
// cached layout signature (`_trace_sig`), per scalar ("scalar", type name), and
// ("alias", i, j, byte distance) for every pair of arrays whose address ranges
// (`_extent`) overlap.  Returns None when an argument is of another kind or an
// array has not cached its signature yet (the Python path then computes it).
PyObject *py_signature(PyObject *, PyObject *pyargs) {
  PyObject *args, *array_type;
  if (!PyArg_ParseTuple(pyargs, "OO", &args, &array_type))
    return nullptr;
  if (!PyTuple_Check(args)) {
    PyErr_SetString(PyExc_TypeError, "args must be a tuple");
    return nullptr;
  }
  const Py_ssize_t n = PyTuple_GET_SIZE(args);
  if (n > 64)
    Py_RETURN_NONE;
  PyObject *items[64 + 64];
  long long lo[64], hi[64];
  int which[64], narr = 0;
  Py_ssize_t count = 0;
  auto fail = [&](bool error) -> PyObject * {
    for (Py_ssize_t i = 0; i < count; ++i)
      Py_DECREF(items[i]);
    if (error)
      return nullptr;
    Py_RETURN_NONE;
  };
  for (Py_ssize_t i = 0; i < n; ++i) {
    PyObject *a = PyTuple_GET_ITEM(args, i);
    if ((PyObject *)Py_TYPE(a) == array_type) {
      PyObject *sig = PyObject_GetAttr(a, sTraceSig);
      if (!sig)
        return fail(true);
      if (sig == Py_None) {
        Py_DECREF(sig);
        return fail(false);
      }
      items[count++] = sig;
      PyObject *ext = PyObject_GetAttr(a, sExtent);
      if (!ext)
        return fail(true);
      if (!PyTuple_Check(ext) || PyTuple_GET_SIZE(ext) != 2) {
        Py_DECREF(ext);
        return fail(false);
      }
      lo[narr] = PyLong_AsLongLong(PyTuple_GET_ITEM(ext, 0));
      hi[narr] = PyLong_AsLongLong(PyTuple_GET_ITEM(ext, 1));
      which[narr++] = (int)i;
      Py_DECREF(ext);
      if (PyErr_Occurred())
        return fail(true);
    } else if (PyBool_Check(a)) {
      items[count++] = Py_BuildValue("(ss)", "scalar", "bool");
    } else if (PyLong_CheckExact(a)) {
      items[count++] = Py_BuildValue("(ss)", "scalar", "int64");
    } else if (PyFloat_CheckExact(a)) {
      items[count++] = Py_BuildValue("(ss)", "scalar", "float64");
    } else {
      return fail(false); // NumPy scalars and anything else: the Python path types them
    }
  }
  // overlapping arrays, in the order the Python implementation lists them:
  // sorted by (lo, hi, index), each array against the later ones that start below its end
  int order[64];
  for (int i = 0; i < narr; ++i)
    order[i] = i;
  for (int i = 1; i < narr; ++i) { // insertion sort: a handful of arrays
    const int x = order[i];
    int j = i - 1;
    while (j >= 0 && (lo[order[j]] > lo[x] || (lo[order[j]] == lo[x] &&
                      (hi[order[j]] > hi[x] || (hi[order[j]] == hi[x] && which[order[j]] > which[x]))))) {
      order[j + 1] = order[j];
      --j;
    }
    order[j + 1] = x;
  }
  for (int k = 0; k + 1 < narr; ++k)
    for (int j = k + 1; j < narr && lo[order[j]] < hi[order[k]]; ++j) {
      if (count >= 128)
        return fail(false);
      items[count++] = Py_BuildValue("(siiL)", "alias", which[order[k]], which[order[j]],
                                     lo[order[j]] - lo[order[k]]);
    }
  PyObject *key = PyTuple_New(count);
  if (!key)
    return fail(true);
  for (Py_ssize_t i = 0; i < count; ++i)
    PyTuple_SET_ITEM(key, i, items[i]); // steals the references
  return key;
}

PyMethodDef kMethods[] = {
    {"init", py_init, METH_VARARGS, "init(launch_address, destroy_event_address[, launch_no_event_address])"},
    {"launch_kernel", py_launch_kernel, METH_VARARGS,
     "launch_kernel(queue, kernel, grid, block, layout, args, tail[, repeat])"},
    {"replay", py_replay, METH_VARARGS, "replay(queue, launches, args)"},
    {"signature", py_signature, METH_VARARGS, "signature(args, array_type)"},
    {nullptr, nullptr, 0, nullptr}};

PyModuleDef kModule = {PyModuleDef_HEAD_INIT, "_fastcall",
                       "Native launch path of numba_mlir_b200 (argument unboxing, GPUParamDesc, launch)", -1,
                       kMethods, nullptr, nullptr, nullptr, nullptr};

} // namespace

PyMODINIT_FUNC PyInit__fastcall(void) {
  sAddr = PyUnicode_InternFromString("_addr");
  sShape = PyUnicode_InternFromString("shape");
  sStrides = PyUnicode_InternFromString("strides");
  sItemsize = PyUnicode_InternFromString("itemsize");
  sTraceSig = PyUnicode_InternFromString("_trace_sig");
  sExtent = PyUnicode_InternFromString("_extent");
  sAlias = PyUnicode_InternFromString("alias");
  return PyModule_Create(&kModule);
}
