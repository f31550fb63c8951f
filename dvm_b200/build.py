"""In-tree build of libdvm_b200.so (host JIT + sm_100a device interpreters + C ABI).

Usage: ``python -m dvm_b200.build [--force]``.  Needs nvcc (CUDA >= 12.8) and g++; cross-compiles for
sm_100a without a GPU.  The shared library lands in ``dvm_b200/lib/`` next to the package so that it
travels with the source tree; nothing is installed outside the tree.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libdvm_b200.so")

SOURCES = [
    "dvm_api.cc",
    "normalize.cc",
    "vcompile.cc",
    "vkernel.cc",
    "partition.cc",
    "stat_fusion.cc",
    "comm.cc",
    "runtime.cu",
    "capi.cu",
    "vm_vector.cu",
    "mm_tcgen05.cu",
    "attn_tcgen05.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    # the interpreters dispatch through dense switches: let ptxas build jump tables (the default threshold
    # of 101 % never does)
    "--jump-table-density=20",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall,-Wno-unused-function",
]
# extra nvcc flags for experiments, e.g. DVM_B200_NVCC_EXTRA="--jump-table-density=101" (later flags win)
NVCC_FLAGS += os.environ.get("DVM_B200_NVCC_EXTRA", "").split()


def _nvcc():
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    path = os.path.join(cuda_home, "bin", "nvcc")
    return path if os.path.exists(path) else "nvcc"


def _newer(src, dst):
    return not os.path.exists(dst) or os.path.getmtime(src) > os.path.getmtime(dst)


def _deps_mtime():
    latest = 0.0
    for d in (CSRC, os.path.join(HERE, "..", "include")):
        for f in os.listdir(d):
            if f.endswith((".h", ".cuh")):
                latest = max(latest, os.path.getmtime(os.path.join(d, f)))
    return latest


def build(force=False, verbose=False):
    os.makedirs(LIB_DIR, exist_ok=True)
    obj_dir = os.path.join(LIB_DIR, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    hdr_time = _deps_mtime()
    jobs = []
    objs = []
    for src in SOURCES:
        sp = os.path.join(CSRC, src)
        op = os.path.join(obj_dir, src.rsplit(".", 1)[0] + ".o")
        objs.append(op)
        if force or _newer(sp, op) or hdr_time > os.path.getmtime(op):
            cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-x", "cu", "-c", sp, "-o", op]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("build failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))
        if verbose:
            sys.stderr.write(r.stderr)
        return r

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(run, jobs))
    if jobs or not os.path.exists(LIB_PATH):
        run([_nvcc(), "-shared", "-o", LIB_PATH] + objs + ["-lcudart", "-ldl"])
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
