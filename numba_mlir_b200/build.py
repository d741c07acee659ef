"""In-tree build of libnumba_mlir_gpu_runtime_cuda.so for sm_100a.

Plays the role of the reference's standalone runtime build
(numba_mlir/setup_helper.py:32-79 builds numba_mlir_gpu_runtime_sycl with icpx):
every .cu under csrc/ is compiled with nvcc for compute_100a/sm_100a and linked,
with a static CUDA runtime, into one shared library placed next to this file,
where the loader looks for it (the reference searches next to the package too,
numba_mlir/mlir/utils.py:17-42).

Run as ``python -m numba_mlir_b200.build [--force] [--verbose]``.
"""

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
BUILD = os.path.join(CSRC, "build")
LIB_NAME = "libnumba_mlir_gpu_runtime_cuda.so"
LIB_PATH = os.path.join(HERE, LIB_NAME)
# CPython extension with the native launch path of the Python front end
# (argument unboxing + GPUParamDesc + launch); plain C++, no CUDA.
FASTCALL_SRC = os.path.join(CSRC, "fastcall", "fastcall.cpp")
FASTCALL_PATH = os.path.join(HERE, "_fastcall.so")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
# -fmad=false: a*b+c is contracted only under fastmath in the reference
# (mlir/lib/Conversion/GpuToGpuRuntime.cpp:2598-2631); CUDA's math library is
# unaffected because it uses explicit fma intrinsics.
COMMON_FLAGS = [
    "-O3",
    "-std=c++17",
    "-lineinfo",
    "-fmad=false",
    "-Xcompiler",
    "-fPIC,-fvisibility=hidden",
    "-Xptxas",
    "-v",
]


def _nvcc():
    path = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(path):
        raise RuntimeError("nvcc not found; the CUDA runtime library cannot be built")
    return path


def _sources():
    out = []
    for root, _dirs, files in os.walk(CSRC):
        if os.path.abspath(root).startswith(BUILD):
            continue
        for f in sorted(files):
            if f.endswith(".cu"):
                out.append(os.path.join(root, f))
    return sorted(out)


def _headers():
    out = []
    for root, _dirs, files in os.walk(CSRC):
        if os.path.abspath(root).startswith(BUILD):
            continue
        for f in files:
            if f.endswith((".h", ".cuh", ".hpp")):
                out.append(os.path.join(root, f))
    out.append(os.path.join(HERE, "..", "include", "numba_mlir_gpu_runtime_cuda.h"))
    return out


def _write_device_header_inc():
    """Embeds kernels/nmb_device.cuh as a string so NVRTC can be given it."""
    src = os.path.join(CSRC, "kernels", "nmb_device.cuh")
    dst = os.path.join(BUILD, "nmb_device_cuh.inc")
    with open(src) as f:
        text = f.read()
    # Adjacent raw string literals; split to stay far below any literal limit.
    chunks = [text[i : i + 8000] for i in range(0, len(text), 8000)]
    body = "\n".join('R"NMBRAW(' + c + ')NMBRAW"' for c in chunks) + "\n"
    old = None
    if os.path.exists(dst):
        with open(dst) as f:
            old = f.read()
    if old != body:
        with open(dst, "w") as f:
            f.write(body)


def build_fastcall(force=False):
    """Compiles the `_fastcall` extension next to the package; returns its path."""
    import sysconfig

    if (not force and os.path.exists(FASTCALL_PATH)
            and os.path.getmtime(FASTCALL_PATH) > os.path.getmtime(FASTCALL_SRC)
            and os.path.getmtime(FASTCALL_PATH) > os.path.getmtime(os.path.abspath(__file__))):
        return FASTCALL_PATH
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        raise RuntimeError("g++ not found; the native launch path cannot be built")
    tmp = FASTCALL_PATH + ".tmp"
    cmd = [cxx, "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-Wall",
           "-I", sysconfig.get_paths()["include"], FASTCALL_SRC, "-o", tmp]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("building _fastcall failed:\n%s\n%s" % (proc.stdout, proc.stderr))
    os.replace(tmp, FASTCALL_PATH)
    return FASTCALL_PATH


def needs_build():
    if not os.path.exists(LIB_PATH):
        return True
    lib_mtime = os.path.getmtime(LIB_PATH)
    deps = _sources() + _headers() + [os.path.abspath(__file__)]
    return any(os.path.getmtime(p) > lib_mtime for p in deps if os.path.exists(p))


def build(force=False, verbose=False):
    """Compiles and links the runtime library (and the `_fastcall` extension);
    returns the library's path."""
    build_fastcall(force)
    if not force and not needs_build():
        return LIB_PATH
    os.makedirs(BUILD, exist_ok=True)
    _write_device_header_inc()
    nvcc = _nvcc()
    lib_mtime = os.path.getmtime(LIB_PATH) if os.path.exists(LIB_PATH) else 0
    header_mtime = max(os.path.getmtime(p) for p in _headers() if os.path.exists(p))

    def compile_one(src):
        rel = os.path.relpath(src, CSRC).replace(os.sep, "_")
        obj = os.path.join(BUILD, rel[:-3] + ".o")
        if (
            not force
            and os.path.exists(obj)
            and os.path.getmtime(obj) > os.path.getmtime(src)
            and os.path.getmtime(obj) > header_mtime
            and os.path.getmtime(obj) > os.path.getmtime(os.path.abspath(__file__))
        ):
            return obj, ""
        cmd = [nvcc, *ARCH_FLAGS, *COMMON_FLAGS, "-I", BUILD, "-I", CSRC, "-c", src, "-o", obj]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(
                "nvcc failed for %s:\n%s\n%s" % (src, proc.stdout, proc.stderr)
            )
        return obj, proc.stderr

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        results = list(pool.map(compile_one, _sources()))
    objs = [r[0] for r in results]
    log = "".join(r[1] for r in results)
    with open(os.path.join(BUILD, "ptxas.log"), "a") as f:
        f.write(log)
    if verbose:
        sys.stderr.write(log)

    tmp = LIB_PATH + ".tmp"
    cmd = [
        nvcc,
        *ARCH_FLAGS,
        "-shared",
        "-cudart",
        "static",
        "-Xcompiler",
        "-fPIC,-fvisibility=hidden",
        "-o",
        tmp,
        *objs,
        "-ldl",
        "-lpthread",
    ]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("link failed:\n%s\n%s" % (proc.stdout, proc.stderr))
    os.replace(tmp, LIB_PATH)
    del lib_mtime
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
