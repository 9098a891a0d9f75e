"""The C++ host mirror of the reference's wrappers (mlx-serve_b200/host/qb200_host.hpp).

CPU: the header compiles with a plain C++17 compiler and links against the C ABI (no GPU call is made).
GPU: the self-test program drives quantizeAffine / qmatmulBits / gatherExpertMm / updateAffine / quantAttention
the way the reference's call sites do and compares every result with the CPU oracle."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "host", "host_selftest.cpp")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _build(tmp_path):
    if shutil.which("g++") is None:
        pytest.skip("g++ not available")
    for lib in (os.path.join(ROOT, "mlx-serve_b200", "libqb200.so"), os.path.join(ROOT, "oracle", "libqoracle.so")):
        if not os.path.exists(lib):
            pytest.fail(f"{lib} is missing: run the build first")
    exe = str(tmp_path / "host_selftest")
    cmd = ["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(ROOT, "mlx-serve_b200", "host"),
           "-I", os.path.join(CUDA, "include"), SRC, "-o", exe,
           "-L", os.path.join(ROOT, "mlx-serve_b200"), "-lqb200", "-L", os.path.join(ROOT, "oracle"), "-lqoracle",
           "-L", os.path.join(CUDA, "lib64"), "-lcudart",
           "-Wl,-rpath," + os.path.join(ROOT, "mlx-serve_b200"), "-Wl,-rpath," + os.path.join(ROOT, "oracle"),
           "-Wl,-rpath," + os.path.join(CUDA, "lib64")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    return exe


def test_host_mirror_compiles_and_links(tmp_path):
    exe = _build(tmp_path)
    r = subprocess.run([exe, "--link-only"], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "linked against qb200" in r.stdout


@pytest.mark.gpu
def test_host_mirror_selftest_on_gpu(tmp_path):
    exe = _build(tmp_path)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert "host self-test passed" in r.stdout
    assert "FAIL" not in r.stdout
