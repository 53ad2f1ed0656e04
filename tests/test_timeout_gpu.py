"""The failure path of the device-side bounded waits, exercised without faulting anything: a self-test kernel waits on
a barrier that nothing completes, with a limit of about a millisecond; the wait gives up, the kernel returns normally,
cct_sync reports CCT_ERR_TIMEOUT and clears the status word, and the context keeps working."""
import numpy as np
import pytest

from tests.parity import assert_close, make_inputs

pytestmark = pytest.mark.gpu


def test_bounded_wait_gives_up_and_the_context_stays_usable(ctx, port):
    from caffecontroll_b200 import capi, conv_layer
    lib = ctx.lib
    assert lib.cct_selftest_bounded_wait(ctx.h, 0) == capi.CCT_ERR_INVALID          # a limit is mandatory
    assert lib.cct_selftest_bounded_wait(ctx.h, 1 << 40) == capi.CCT_ERR_INVALID    # and cannot exceed the kernels' own
    capi.check(lib.cct_selftest_bounded_wait(ctx.h, 2_000_000), "cct_selftest_bounded_wait", ctx.h)  # ~1 ms of SM clock
    assert lib.cct_sync(ctx.h) == capi.CCT_ERR_TIMEOUT
    assert b"0x7e57" in lib.cct_last_error_string(ctx.h)
    assert lib.cct_sync(ctx.h) == capi.CCT_OK  # the status word was cleared by the failing sync
    # the next convolution call runs as usual
    B, D, n, o, k, s, p, g = 2, 8, 9, 12, 5, 1, 2, 2
    X, W, b, dY = make_inputs(77, B, D, n, o, k, s, p, g)
    Y, dX, dW, db, _ = conv_layer(ctx, X, W, b, dY, k, s, p, g, algo=capi.ALGO_UMMA_3XTF32)
    assert_close(Y, port.conv_forward(X, W, b, k, s, p, g), "Y after a timed-out wait")
    dXr, dWr, dbr = port.conv_backward(X, W, dY, k, s, p, g)
    for a, r, name in ((dX, dXr, "dX"), (dW, dWr, "dW"), (db, dbr, "db")):
        assert_close(a, r, name + " after a timed-out wait")


def test_calls_refuse_to_queue_behind_a_pending_timeout(ctx):
    """Between the wait giving up and the next cct_sync, convolution calls return CCT_ERR_TIMEOUT instead of piling up."""
    import ctypes as C
    import time
    from caffecontroll_b200 import capi
    lib = ctx.lib
    desc = capi.ConvDesc(1, 2, 8, 4, 3, 1, 1, 1, 1, capi.ALGO_UMMA_3XTF32)
    plan = C.c_void_p()
    capi.check(lib.cct_conv_plan_create(ctx.h, C.byref(desc), C.byref(plan)), "plan", ctx.h)
    buf = ctx.malloc(4096)
    capi.check(lib.cct_selftest_bounded_wait(ctx.h, 1_000_000), "selftest", ctx.h)
    time.sleep(0.2)  # the kernel has long returned; the status word (mapped host memory) is set
    vp = C.c_void_p
    assert lib.cct_conv_forward(plan, vp(buf), vp(buf), vp(buf), vp(buf), 0) == capi.CCT_ERR_TIMEOUT
    assert lib.cct_sync(ctx.h) == capi.CCT_ERR_TIMEOUT
    assert lib.cct_sync(ctx.h) == capi.CCT_OK
    capi.check(lib.cct_conv_plan_destroy(plan), "destroy", ctx.h)
    ctx.free(buf)
