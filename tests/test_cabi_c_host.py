"""A host program in C against the public header: the header compiles as
pedantic C99, the program links to the library, and (on a GPU) runs the call
sequence of the reference's generated host code end to end."""

import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cabi", "host_example.c")


@pytest.fixture(scope="module")
def host_binary(tmp_path_factory, runtime_lib):
    if shutil.which("gcc") is None:
        pytest.skip("no C compiler")
    libdir = os.path.join(ROOT, "numba_mlir_b200")
    exe = str(tmp_path_factory.mktemp("cabi") / "host_example")
    cmd = ["gcc", "-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic", "-I", os.path.join(ROOT, "include"), SRC,
           "-o", exe, "-L", libdir, "-lnumba_mlir_gpu_runtime_cuda", f"-Wl,-rpath,{libdir}"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr
    return exe


def test_header_is_c99_and_error_paths_need_no_device(host_binary):
    proc = subprocess.run([host_binary, "--no-device"], capture_output=True, text=True, timeout=120)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "ok (no device)" in proc.stdout


@pytest.mark.gpu
def test_c_host_runs_the_generated_code_call_sequence(host_binary):
    proc = subprocess.run([host_binary], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert proc.stdout.startswith("ok: 307200 elements")
