"""CPU tests of the drop-in boundary: the shared library loads, exports every symbol the header declares, and
argument validation works without touching a GPU."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from caffecontroll_b200 import _build, capi
    _build.build()
    return capi.load()


def _declared():
    with open(os.path.join(ROOT, "include", "cct_b200.h")) as f:
        text = re.sub(r"/\*.*?\*/", "", f.read(), flags=re.S)
    return sorted(set(re.findall(r"\b(cct_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_list_the_same_symbols():
    from caffecontroll_b200 import capi
    assert _declared() == sorted(capi.EXPORTS)


def test_library_exports_every_declared_symbol(lib):
    for name in _declared():
        assert getattr(lib, name) is not None, name


def test_out_size_and_descriptor_validation(lib):
    from caffecontroll_b200 import capi
    m = C.c_int()
    d = capi.ConvDesc(256, 3, 227, 96, 11, 4, 0, 1, 1, 0)
    assert lib.cct_conv_out_size(C.byref(d), C.byref(m)) == capi.CCT_OK and m.value == 55
    d = capi.ConvDesc(256, 96, 27, 256, 5, 1, 2, 2, 1, 0)
    assert lib.cct_conv_out_size(C.byref(d), C.byref(m)) == capi.CCT_OK and m.value == 27
    for bad in (capi.ConvDesc(0, 3, 227, 96, 11, 4, 0, 1, 1, 0),    # empty batch
                capi.ConvDesc(4, 3, 5, 8, 7, 1, 0, 1, 1, 0),        # kernel larger than padded input
                capi.ConvDesc(4, 3, 9, 8, 3, 1, 0, 2, 1, 0),        # depth not divisible by groups
                capi.ConvDesc(4, 4, 9, 8, 3, 0, 0, 1, 1, 0)):       # zero stride
        assert lib.cct_conv_out_size(C.byref(bad), C.byref(m)) == capi.CCT_ERR_INVALID


def test_null_arguments_are_rejected_not_crashing(lib):
    from caffecontroll_b200 import capi
    assert lib.cct_ctx_create(0, None) == capi.CCT_ERR_INVALID
    assert lib.cct_sync(None) == capi.CCT_ERR_INVALID
    assert lib.cct_conv_forward(None, None, None, None, None, 0) == capi.CCT_ERR_INVALID
    assert lib.cct_conv_backward(None, None, None, None, None, None, None) == capi.CCT_ERR_INVALID
    assert lib.cct_sgd_step(None, 4, None, None, None, 0.1, 0.9, 0.0) == capi.CCT_ERR_INVALID


def test_context_creation_without_a_gpu_fails_with_a_status(lib):
    from caffecontroll_b200 import capi
    n = C.c_int(-1)
    rc = lib.cct_device_count(C.byref(n))
    if rc == capi.CCT_OK and n.value > 0:
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    assert lib.cct_ctx_create(0, C.byref(h)) != capi.CCT_OK and not h.value
