"""The C++ expert-parallel drivers (qwen4-thor_b200/host/q4t/parallel/ep_driver.h: NCCL +
the C ABI, no Python in the loop): they must compile and link here, and on a GPU box one
process per GPU (two when two devices are visible, otherwise a single rank, which still runs
every NCCL call) must reproduce the single-GPU layer bit for bit."""
import os
import subprocess
import tempfile

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "tests", "cpp", "ep_driver_test")


def _nccl_flags():
    """System NCCL if its header is installed, else the copy bundled with the nvidia-nccl wheel."""
    if os.path.exists("/usr/include/nccl.h"):
        return [], ["-lnccl"]
    try:
        import nvidia.nccl as n
        base = os.path.dirname(n.__file__)
        lib = os.path.join(base, "lib")
        return [f"-I{os.path.join(base, 'include')}"], [f"-L{lib}", "-l:libnccl.so.2", f"-Wl,-rpath,{lib}"]
    except ImportError:
        return None, None


def _build():
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    pkg = os.path.join(ROOT, "qwen4-thor_b200")
    inc, link = _nccl_flags()
    if inc is None:
        pytest.skip("no NCCL header on this machine")
    cmd = ["g++", "-std=c++20", "-O1", "-Wall", "-pthread", f"-I{cuda}/include", f"-I{ROOT}/include", f"-I{pkg}/host", *inc,
           os.path.join(ROOT, "tests", "cpp", "ep_driver_test.cpp"), "-o", EXE,
           f"-L{pkg}", "-lq4t_moe_b200", f"-Wl,-rpath,{pkg}", f"-L{cuda}/lib64", "-lcudart", *link]
    return subprocess.run(cmd, capture_output=True, text=True)


def test_ep_driver_compiles_and_links(q4t):
    if not os.path.exists(q4t.LIB_PATH):
        pytest.skip("library not built")
    r = _build()
    assert r.returncode == 0, r.stderr


@pytest.mark.gpu
def test_ep_driver_runs_on_gpus(q4t, gpu_lib):
    import torch
    if not os.path.exists(EXE):
        r = _build()
        assert r.returncode == 0, r.stderr
    world = 2 if torch.cuda.device_count() >= 2 else 1
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    with tempfile.TemporaryDirectory() as tmp:
        id_file = os.path.join(tmp, "nccl_id")
        procs = [subprocess.Popen([EXE, str(r), str(world), id_file], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                  text=True, env=env) for r in range(world)]
        outs = []
        for p in procs:
            try:
                out, _ = p.communicate(timeout=600)
            except subprocess.TimeoutExpired:
                for q in procs:
                    q.kill()
                raise
            outs.append((p.returncode, out))
    for r, (rc, out) in enumerate(outs):
        assert rc == 0 and f"ep_driver_test PASS rank {r} of {world}" in out, out[-3000:]
