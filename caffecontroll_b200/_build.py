"""Build recipe for libcct_b200.so: every .cu under csrc/ compiled for sm_100a (one object per source, in parallel,
rebuilt only when the source or a header is newer) and linked into one shared library that sits next to this file
(in-tree, so it travels with the source snapshot)."""
import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libcct_b200.so")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _headers():
    return glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh")) + \
        glob.glob(os.path.join(HERE, "..", "include", "*.h"))


def up_to_date():
    if not os.path.exists(LIB):
        return False
    t = os.path.getmtime(LIB)
    return all(os.path.getmtime(f) <= t for f in sources() + _headers())


def build(force=False, verbose_ptxas=False):
    if not force and up_to_date():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    os.makedirs(OBJ, exist_ok=True)
    hdr_time = max([os.path.getmtime(h) for h in _headers()] + [0.0])

    def compile_one(src):
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        if not force and not verbose_ptxas and os.path.exists(obj) and \
                os.path.getmtime(obj) >= max(os.path.getmtime(src), hdr_time):
            return obj
        cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose_ptxas else []) + ["-c", "-o", obj, src]
        print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, sources()))
    tmp = LIB + ".tmp"  # written beside the target, then renamed: a reader never sees a half-written library
    # libdl: the NCCL entry points are looked up at run time (the library has no link-time dependency on NCCL)
    cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", tmp] + objs + ["-ldl"]
    print(" ".join(cmd), flush=True)
    subprocess.check_call(cmd)
    os.replace(tmp, LIB)
    return LIB


HOST_TEST = os.path.join(HERE, "host", "host_selftest")


def build_host_selftest(force=False):
    """The C++ bridge mirror's self-test program (g++ only: it sees nothing but the C ABI)."""
    src = os.path.join(HERE, "host", "host_selftest.cpp")
    hdr = os.path.join(HERE, "host", "cct_host.h")
    if not force and os.path.exists(HOST_TEST) and all(
            os.path.getmtime(f) <= os.path.getmtime(HOST_TEST) for f in (src, hdr, LIB)):
        return HOST_TEST
    cmd = ["g++", "-std=c++14", "-O2", "-Wall", "-o", HOST_TEST, src, "-L" + HERE, "-lcct_b200", "-Wl,-rpath,$ORIGIN/..",
           "-pthread"]
    print(" ".join(cmd), flush=True)
    subprocess.check_call(cmd)
    return HOST_TEST


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose_ptxas="-v" in sys.argv)
    build_host_selftest(force="--force" in sys.argv)
