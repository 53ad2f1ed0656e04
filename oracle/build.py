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


def reference_root():
    """The reference source tree: the directory CCT_REFERENCE_ROOT names, else a checkout called `reference` beside
    this repository (absent on machines that only run the prebuilt checkers)."""
    return os.environ.get(REF_ENV) or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


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
    ref = reference_root()
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


def _read_floats(path):
    import numpy as np
    with open(path) as f:
        return np.array(f.read().split(), dtype=np.float32)


def build_adaptor_test(force=False):
    """The reference-tree adaptor (caffecontroll_b200/host/reference_adaptor/*.h) compiled against the reference's own
    headers in place, with the oracle's three shim headers, into oracle/_ref/adaptor_fixture_test; beside it the
    reference's text fixtures of tests/test_parallelized_convolution.cpp converted to raw fp32 files (git-ignored, they
    travel with the built program).  Only possible where the reference tree is mounted."""
    ref = reference_root()
    src_dir = os.path.join(ref, "src")
    out_dir = os.path.join(HERE, "_ref")
    exe = os.path.join(out_dir, "adaptor_fixture_test")
    if not os.path.isdir(src_dir):
        return exe if os.path.exists(exe) else None
    root = os.path.dirname(HERE)
    adaptor = os.path.join(root, "caffecontroll_b200", "host", "reference_adaptor")
    main_cpp = os.path.join(root, "tests", "adaptor_fixture_main.cpp")
    lib_dir = os.path.join(root, "caffecontroll_b200")
    deps = [main_cpp, os.path.join(root, "include", "cct_b200.h")] + glob.glob(os.path.join(adaptor, "*.h")) + \
        glob.glob(os.path.join(HERE, "shim", "**", "*.h*"), recursive=True)
    os.makedirs(out_dir, exist_ok=True)
    if force or not _newer(exe, deps):
        blas = scipy_openblas()
        ref_srcs = [os.path.join(src_dir, p) for p in
                    ("sched/DeviceDriver_CPU.cpp", "util.cpp", "timer.cpp", "DeepNetConfig.cpp")]
        _run(["g++", "-std=c++11", "-O2", "-w", "-pthread", "-D_USE_OPENBLAS", "-include", "climits", "-include", "algorithm",
              "-I" + os.path.join(HERE, "shim", "inc"), "-I" + src_dir, "-I" + adaptor, "-I" + os.path.join(root, "include"),
              "-o", exe, main_cpp] + ref_srcs +
             [blas, "-Wl,-rpath," + os.path.dirname(blas), "-L" + lib_dir, "-lcct_b200", "-Wl,-rpath,$ORIGIN/../../caffecontroll_b200"])
    fix = os.path.join(out_dir, "conv_fixture")
    tests = os.path.join(ref, "tests")
    names = {"X": "input/conv_forward_in.txt", "W_fwd": "input/conv_model.txt", "W_bwd": "input/conv_backward_model.txt",
             "b": "input/conv_bias_in.txt", "Y": "output/conv_forward.txt", "dX": "output/conv_backward.txt",
             "b_new": "output/conv_bias.txt", "W_new": "output/conv_weights.txt"}
    if os.path.isdir(tests) and (force or not os.path.exists(os.path.join(fix, "W_new.bin"))):
        os.makedirs(fix, exist_ok=True)
        for key, rel in names.items():
            _read_floats(os.path.join(tests, rel)).tofile(os.path.join(fix, key + ".bin"))
    return exe


def main():
    force = "--force" in sys.argv
    print("port     :", build_port(force))
    print("reference:", build_reference(force))
    print("adaptor  :", build_adaptor_test(force))


if __name__ == "__main__":
    main()
