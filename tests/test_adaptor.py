"""The reference-tree adaptor (caffecontroll_b200/host/reference_adaptor/): class B200Driver : public DeviceDriver, the
AbstractBridge and ConvolutionBridge specialisations for it, and ParallelizedBridge_B200 with the scheduler-facing
virtuals - compiled against the reference's own headers in place (CPU check, where the reference tree is mounted), and run
on the reference's own parallelized-convolution fixture on a GPU (the built program and the converted fixture files
travel under oracle/_ref/)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
EXE = os.path.join(ROOT, "oracle", "_ref", "adaptor_fixture_test")
FIXTURE = os.path.join(ROOT, "oracle", "_ref", "conv_fixture")


def _build():
    from caffecontroll_b200 import _build
    from oracle import build as obuild
    _build.build()
    return obuild.build_adaptor_test()


def test_adaptor_compiles_against_the_reference_headers():
    from oracle import build as obuild
    ref = obuild.reference_root()
    if not os.path.isdir(os.path.join(ref, "src")):
        pytest.skip("the reference tree is not mounted here")
    exe = _build()
    assert exe and os.path.exists(exe)
    out = subprocess.run([exe, "--compile-check"], capture_output=True, text=True)
    assert out.returncode == 0 and "compiled against the reference headers" in out.stdout
    with open(os.path.join(ROOT, "caffecontroll_b200", "host", "reference_adaptor", "DeviceDriver_B200.h")) as f:
        text = f.read()
    # every pure virtual of src/sched/DeviceDriver.h:76-86, 197-206 is implemented
    for name in ("choose_ptr", "get_device_pointer", "void malloc", "void free", "void memcpy", "void memset", "math_saxpy",
                 "math_saxpby", "set_num_threads", "void sgemm"):
        assert name in text, name


@pytest.mark.gpu
def test_reference_fixture_through_the_adaptor():
    if not (os.path.exists(EXE) and os.path.exists(os.path.join(FIXTURE, "W_new.bin"))):
        pytest.skip("oracle/_ref/adaptor_fixture_test was not built (needs the reference tree at build time)")
    out = subprocess.run([EXE, FIXTURE], capture_output=True, text=True, timeout=300)
    print(out.stdout, out.stderr)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "adaptor fixture test ok" in out.stdout
