"""The C++ shims that rebuild the reference's operator signatures on the C ABI:
they must compile as host C++ (CPU test) and run end to end on a GPU."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "tests", "cpp", "shim_test")


def _build():
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    pkg = os.path.join(ROOT, "qwen4-thor_b200")
    cmd = ["g++", "-std=c++20", "-O1", "-Wall", "-pthread", f"-I{cuda}/include", f"-I{ROOT}/include", f"-I{pkg}/host",
           os.path.join(ROOT, "tests", "cpp", "shim_test.cpp"), "-o", EXE,
           f"-L{pkg}", "-lq4t_moe_b200", f"-Wl,-rpath,{pkg}", f"-L{cuda}/lib64", "-lcudart"]
    return subprocess.run(cmd, capture_output=True, text=True)


def test_shims_compile_and_link(q4t):
    if not os.path.exists(q4t.LIB_PATH):
        pytest.skip("library not built")
    r = _build()
    assert r.returncode == 0, r.stderr


@pytest.mark.gpu
def test_shims_run_on_gpu(q4t, gpu_lib):
    if not os.path.exists(EXE):
        r = _build()
        assert r.returncode == 0, r.stderr
    r = subprocess.run([EXE], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "shim_test PASS" in r.stdout, r.stdout + r.stderr
