"""The C++ class API (include/dvm.h) from a C++ client: tests/cpp/client.cc is compiled against the header, linked with
libdvm_b200.so and run, the way a user of the reference's `dvm::Kernel` links libdvm.a (include/dvm.h:236-648)."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_DIR = os.path.join(ROOT, "dvm_b200", "lib")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def build(tmp_path, with_cuda):
    exe = str(tmp_path / ("client_cuda" if with_cuda else "client"))
    cmd = ["g++", "-std=c++17", "-O1", "-I" + os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "cpp", "client.cc"),
           "-o", exe, "-L" + LIB_DIR, "-ldvm_b200", "-Wl,-rpath," + LIB_DIR]
    if with_cuda:
        cmd += ["-DWITH_CUDA", "-I" + os.path.join(CUDA, "include"), "-L" + os.path.join(CUDA, "lib64"), "-lcudart",
                "-Wl,-rpath," + os.path.join(CUDA, "lib64")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    return exe


def test_cpp_client_builds_infers_and_compiles(tmp_path):
    from dvm_b200 import build as lib_build
    lib_build.build()
    r = subprocess.run([build(tmp_path, False), "dry"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "DRY OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
    assert "vmain.sm100" in r.stdout and "ReduceSum" in r.stdout


@pytest.mark.gpu
def test_cpp_client_launches_and_relocates(tmp_path):
    r = subprocess.run([build(tmp_path, True), "run"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "RUN OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
