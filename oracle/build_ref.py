"""Builds the reference's own CUDA backend (mindspore-ai/dvm, `DVM_ARCH=gpu`) into oracle/_ref/ for cross-checking.

TEST INFRASTRUCTURE ONLY.  The sources are compiled where they lie (the read-only reference tree: the directory given on the
command line, else DVM_REFERENCE_DIR, else a directory named `reference` beside this repository); nothing is copied into this repository and every output goes to oracle/_ref/, which is git-ignored.
The recipe restates the GPU branch of the reference's Makefile (Makefile:7-14, 84-103): g++ on the host sources with
-DDVM_ARCH_GPU, nvcc on src/vm_gpu.cu for sm_100a, one shared pybind11 module `_dvm_py`.  The reference's GPU backend
executes vector kernels only (src/system.cc:290-294), so it cross-checks the elementwise / reduce graphs, not MatMul.

Usage: python -m oracle.build_ref [reference_dir]
"""
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

HOST_SOURCES = ["ops.cc", "ops_m.cc", "ops_c.cc", "kernel.cc", "xkernel.cc", "gkernel.cc", "code.cc", "dvm.cc", "schedule.cc",
                "pass.cc", "utils.cc", "vf_fusion.cc", "system.cc", "pybind_api.cc", "dry_run.cc"]


def module_path():
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return os.path.join(OUT, "_dvm_py" + suffix)


def find_reference():
    """The reference tree: DVM_REFERENCE_DIR when set, else a directory named `reference` beside this repository."""
    env = os.environ.get("DVM_REFERENCE_DIR")
    if env:
        return env
    return os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


DEFAULT_REFERENCE = find_reference()


def build(ref=DEFAULT_REFERENCE, force=False):
    """Returns the path of the built module, or None when the reference tree or a toolchain piece is missing."""
    src = os.path.join(ref, "src")
    if not os.path.isdir(src):
        return None
    target = module_path()
    if os.path.exists(target) and not force:
        return target
    try:
        import pybind11
    except ImportError:
        return None
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    nvcc = os.path.join(cuda, "bin", "nvcc")
    os.makedirs(OUT, exist_ok=True)
    inc = ["-I" + os.path.join(ref, "include"), "-I" + src, "-I" + os.path.join(cuda, "include"),
           "-I" + pybind11.get_include(), "-I" + sysconfig.get_paths()["include"]]
    cflags = ["--std=c++17", "-Wall", "-fPIC", "-fvisibility=hidden", "-DDVM_ARCH_GPU", "-Wno-array-bounds", "-O2"]
    jobs, objs = [], []
    for name in HOST_SOURCES:
        obj = os.path.join(OUT, name[:-3] + ".o")
        objs.append(obj)
        jobs.append(["g++", "-c"] + cflags + inc + [os.path.join(src, name), "-o", obj])
    vm = os.path.join(OUT, "vm.o")
    objs.append(vm)
    jobs.append([nvcc, "-c", "-O2", "--std=c++17", "-DDVM_ARCH_GPU", "-gencode", "arch=compute_100a,code=sm_100a",
                 "--jump-table-density=60", "-Xcompiler", "-fPIC"] + inc[:2] + [os.path.join(src, "vm_gpu.cu"), "-o", vm])

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True, cwd=OUT)
        if r.returncode != 0:
            raise RuntimeError("reference build failed: %s\n%s" % (" ".join(cmd), r.stderr[-2000:]))

    with ThreadPoolExecutor(max_workers=8) as ex:
        list(ex.map(run, jobs))
    # -Bsymbolic: the module keeps using its own dvm:: symbols when this library is loaded in the same process
    run(["g++", "-shared", "-Wl,-Bsymbolic"] + objs + ["-L" + os.path.join(cuda, "lib64"), "-lcudart", "-o", target])
    for obj in objs:   # only the module travels to the GPU box
        os.remove(obj)
    return target


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 and not sys.argv[1].startswith("-") else DEFAULT_REFERENCE, force="--force" in sys.argv))
