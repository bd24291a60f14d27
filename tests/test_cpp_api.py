"""The C++ `ctd::` surface (include/ctd/*.h over include/ctd/b200/*.hpp): it compiles and links against the
C-ABI library on any host; on a B200 the case lists in tests/cpp/ (the reference's op tests, and its
training-loop idiom against the step engine) run and must pass."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "emberlm_b200")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


PROGRAMS = ["test_ctd_api", "test_ctd_train_loop", "test_ctd_autograd"]


def _build(tmp_path, name):
    exe = str(tmp_path / name)
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-Wextra", "-Werror",
           "-I", os.path.join(ROOT, "include"), "-I", os.path.join(CUDA, "include"),
           os.path.join(ROOT, "tests", "cpp", name + ".cpp"), "-o", exe,
           "-L", PKG, "-lctdk", "-L", os.path.join(CUDA, "lib64"), "-lcudart",
           "-Wl,-rpath," + PKG, "-Wl,-rpath," + os.path.join(CUDA, "lib64")]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-4000:]
    return exe


@pytest.mark.parametrize("name", PROGRAMS)
def test_header_compiles_and_links(tmp_path, name):
    assert os.path.exists(os.path.join(PKG, "libctdk.so")), "build the library first: python -m emberlm_b200.build"
    _build(tmp_path, name)


@pytest.mark.gpu
@pytest.mark.parametrize("name", PROGRAMS)
def test_cpp_cases_pass_on_gpu(tmp_path, name):
    exe = _build(tmp_path, name)
    res = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    print(res.stdout[-6000:])
    assert res.returncode == 0, res.stdout[-6000:] + res.stderr[-2000:]
    assert "0 failed" in res.stdout
