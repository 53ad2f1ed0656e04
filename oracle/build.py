"""TEST INFRASTRUCTURE — build recipe for the two CPU checkers under oracle/.

1. oracle/liboracle.so   : the plain-C restatement (conv_oracle.c), always built.
2. oracle/_ref/libcct_ref.so : the reference's own CPU code (CPUDriver, ConvolutionBridge, ParallelizedBridge,
   MaxPoolingBridge, ReLUBridge) compiled in place from the reference source tree, only when that tree is
   present.  Nothing is copied from it; the three headers under oracle/shim/ stand in for cblas.h, boost/random.hpp
   and the protoc output the tree expects.  BLAS is the LP64 OpenBLAS bundled inside the scipy wheel.

Flags follow the reference's test_debug target: no -Ofast, no -D_FASTPOW (its product build's approximate pow).
"""
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_ENV = "CCT_REFERENCE_ROOT"
DEFAULT_REF = "/root/reference"


def _run(cmd):
    print(" ".join(cmd), flush=True)
    subprocess.check_call(cmd)


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources if os.path.exists(s))


def scipy_openblas():
    import scipy  # noqa: F401  (only to locate the wheel)

    libs = os.path.join(os.path.dirname(os.path.dirname(scipy.__file__)), "scipy.libs")
    hits = sorted(glob.glob(os.path.join(libs, "libscipy_openblas*.so")))
    if not hits:
        raise RuntimeError("no libscipy_openblas*.so under %s" % libs)
    return hits[0]


def build_port(force=False):
    src = os.path.join(HERE, "conv_oracle.c")
    out = os.path.join(HERE, "liboracle.so")
    if force or not _newer(out, [src]):
        _run(["gcc", "-O3", "-march=native", "-fopenmp", "-fPIC", "-shared", "-std=c11", "-Wall",
              "-fno-fast-math", "-o", out, src, "-lm"])
    return out


def build_reference(force=False):
    ref = os.environ.get(REF_ENV, DEFAULT_REF)
    src_dir = os.path.join(ref, "src")
    out_dir = os.path.join(HERE, "_ref")
    out = os.path.join(out_dir, "libcct_ref.so")
    if not os.path.isdir(src_dir):
        return out if os.path.exists(out) else None
    wrapper = os.path.join(HERE, "ref_wrapper.cpp")
    shims = glob.glob(os.path.join(HERE, "shim", "**", "*.h*"), recursive=True)
    if not force and _newer(out, [wrapper] + shims):
        return out
    os.makedirs(out_dir, exist_ok=True)
    blas = scipy_openblas()
    ref_srcs = [os.path.join(src_dir, p) for p in
                ("sched/DeviceDriver_CPU.cpp", "util.cpp", "timer.cpp", "DeepNetConfig.cpp")]
    _run(["g++", "-std=c++11", "-O3", "-march=native", "-fPIC", "-shared", "-w", "-pthread",
          "-D_USE_OPENBLAS", "-include", "climits", "-include", "algorithm",
          "-I" + os.path.join(HERE, "shim", "inc"), "-I" + src_dir,
          "-o", out, wrapper] + ref_srcs +
         [blas, "-Wl,-rpath," + os.path.dirname(blas)])
    return out


def main():
    force = "--force" in sys.argv
    print("port     :", build_port(force))
    print("reference:", build_reference(force))


if __name__ == "__main__":
    main()
