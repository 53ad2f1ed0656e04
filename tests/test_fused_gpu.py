"""cct_conv_backward_fused against the chain the reference runs as separate bridges: MaxPoolingBridge::backward ->
ReLUBridge::backward -> ConvolutionBridge::backward (-> ReLUBridge::backward of the layer in front).  The oracle is the
CPU restatement of those bridges; convolution results are held to max-norm relative error <= 1e-4, and the positions
the ReLU mask zeroes must be zero exactly."""
import ctypes as C

import numpy as np
import pytest

from caffecontroll_b200 import capi
from caffecontroll_b200.bridge import LogicalCube
from tests.parity import TOL, assert_close

pytestmark = pytest.mark.gpu

# (B, D, n, o, k, s, p, g, pool_k, pool_s); the last one is the CaffeNet conv2 geometry at a small batch
SHAPES = [
    (2, 4, 13, 6, 3, 1, 1, 1, 3, 2),
    (3, 6, 12, 8, 5, 1, 2, 2, 2, 2),
    (2, 3, 23, 16, 7, 2, 0, 1, 3, 2),
    (4, 96, 27, 256, 5, 1, 2, 2, 3, 2),
]


def _run(ctx, port, shape, algo):
    B, D, n, o, k, s, p, g, pk, ps = shape
    m = (n + 2 * p - k) // s + 1
    mp = (m - pk) // ps + 1
    rng = np.random.default_rng(1000 * 3 + n)
    X = np.maximum(rng.standard_normal((B, D, n, n), dtype=np.float32), 0)  # post-ReLU input, as in CaffeNet
    W = (0.01 * rng.standard_normal((o, D // g, k, k))).astype(np.float32)
    bias = np.ones(o, np.float32) * 0.1
    dP = rng.standard_normal((B, o, mp, mp), dtype=np.float32)

    lib, vp = ctx.lib, C.c_void_p
    desc = capi.ConvDesc(B, D, n, o, k, s, p, g, 1, algo)
    plan = C.c_void_p()
    capi.check(lib.cct_conv_plan_create(ctx.h, C.byref(desc), C.byref(plan)), "plan", ctx.h)
    capi.check(lib.cct_conv_plan_reserve_fusion(plan), "reserve", ctx.h)
    cX, cW, cb, cdP = (LogicalCube.from_numpy(ctx, a) for a in (X, W, bias, dP))
    cY = LogicalCube(ctx, m, m, o, B)
    cPool, cidx = LogicalCube(ctx, mp, mp, o, B), LogicalCube(ctx, mp, mp, o, B, np.int32)
    cdX, cdW, cdb = LogicalCube(ctx, n, n, D, B), LogicalCube(ctx, k, k, D // g, o), LogicalCube(ctx, 1, 1, o, 1)
    # forward with the ReLU folded in, then the pooling bridge
    capi.check(lib.cct_conv_forward(plan, vp(cX.ptr), vp(cW.ptr), vp(cb.ptr), vp(cY.ptr), 1), "fwd", ctx.h)
    capi.check(lib.cct_maxpool_forward(ctx.h, vp(cY.ptr), vp(cPool.ptr), vp(cidx.ptr), B * o, m, pk, ps), "pool", ctx.h)
    ctx.sync()
    Yg = cY.download()
    out = {}
    for mask_dx in (0, 1):
        f = capi.BwdFusion(cY.ptr, cidx.ptr, cdP.ptr, pk, ps, mask_dx)
        capi.check(lib.cct_conv_backward_fused(plan, vp(cX.ptr), vp(cW.ptr), None, C.byref(f), vp(cdX.ptr), vp(cdW.ptr),
                                               vp(cdb.ptr)), "bwd fused", ctx.h)
        ctx.sync()
        out[mask_dx] = (cdX.download(), cdW.download(), cdb.download())
    # the same with the ReLU mask taken from the pooled tensor instead of the layer's output: bit-identical
    f = capi.BwdFusion(None, cidx.ptr, cdP.ptr, pk, ps, 0, cPool.ptr)
    capi.check(lib.cct_conv_backward_fused(plan, vp(cX.ptr), vp(cW.ptr), None, C.byref(f), vp(cdX.ptr), vp(cdW.ptr),
                                           vp(cdb.ptr)), "bwd fused, pooled mask", ctx.h)
    ctx.sync()
    for got, want in zip((cdX.download(), cdW.download(), cdb.download()), out[0]):
        assert np.array_equal(got, want)
    # the ReLU mask alone, on a caller-supplied dY
    _, idx0 = port.maxpool_forward(Yg, pk, ps)
    cdY = LogicalCube.from_numpy(ctx, port.relu_backward(Yg, port.maxpool_backward(dP, idx0, m)))
    f = capi.BwdFusion(None, None, None, 0, 0, 1)
    capi.check(lib.cct_conv_backward_fused(plan, vp(cX.ptr), vp(cW.ptr), vp(cdY.ptr), C.byref(f), vp(cdX.ptr),
                                           vp(cdW.ptr), vp(cdb.ptr)), "bwd relu only", ctx.h)
    ctx.sync()
    only_relu = cdX.download()
    idx_gpu = cidx.download()
    capi.check(lib.cct_conv_plan_destroy(plan), "destroy", ctx.h)
    for c in (cX, cW, cb, cdP, cY, cPool, cidx, cdX, cdW, cdb, cdY):
        c.free()

    # Oracle chain, started from the forward output the device produced (the forward pass has its own parity tests;
    # starting from the oracle's own forward would let 1e-6 differences flip the winner of a near-tie in a window).
    _, idxr = port.maxpool_forward(Yg, pk, ps)
    dAr = port.maxpool_backward(dP, idxr, m)
    dYr = port.relu_backward(Yg, dAr)
    dXr, dWr, dbr = port.conv_backward(X, W, dYr, k, s, p, g)
    dXr_masked = port.relu_backward(X, dXr)
    assert np.array_equal(idx_gpu, idxr)
    dX0, dW0, db0 = out[0]
    assert_close(dX0, dXr, "dX (pool+relu on the output side)")
    assert_close(dW0.reshape(dWr.shape), dWr, "dW")
    assert_close(db0.reshape(dbr.shape), dbr, "db")
    dX1, dW1, db1 = out[1]
    assert_close(dX1, dXr_masked, "dX with the input-side ReLU mask")
    assert np.all(dX1[X <= 0] == 0.0)
    assert np.array_equal(dW1, dW0) and np.array_equal(db1, db0)
    assert_close(only_relu, dXr_masked, "dX, ReLU mask only")
    assert np.all(only_relu[X <= 0] == 0.0)


@pytest.mark.parametrize("algo", [capi.ALGO_SIMT_FP32, capi.ALGO_UMMA_3XTF32])
@pytest.mark.parametrize("shape", SHAPES)
def test_fused_backward_matches_bridge_chain(ctx, port, shape, algo):
    if algo == capi.ALGO_SIMT_FP32 and shape[0] * shape[1] * shape[3] > 4000:
        pytest.skip("the direct fp32 kernels are the small-shape fallback")
    _run(ctx, port, shape, algo)


def test_fused_backward_argument_checks(ctx):
    lib, vp = ctx.lib, C.c_void_p
    desc = capi.ConvDesc(1, 2, 8, 4, 3, 1, 1, 1, 1, capi.ALGO_AUTO)
    plan = C.c_void_p()
    capi.check(lib.cct_conv_plan_create(ctx.h, C.byref(desc), C.byref(plan)), "plan", ctx.h)
    buf = LogicalCube(ctx, 8, 8, 4, 4)
    f = capi.BwdFusion(None, None, buf.ptr, 3, 2, 0)  # dP without A / idx
    rc = lib.cct_conv_backward_fused(plan, vp(buf.ptr), vp(buf.ptr), None, C.byref(f), None, vp(buf.ptr), vp(buf.ptr))
    assert rc == capi.CCT_ERR_INVALID
    f = capi.BwdFusion(buf.ptr, buf.ptr, buf.ptr, 3, 2, 0)  # a pooled gradient without cct_conv_plan_reserve_fusion
    rc = lib.cct_conv_backward_fused(plan, vp(buf.ptr), vp(buf.ptr), None, C.byref(f), None, vp(buf.ptr), vp(buf.ptr))
    assert rc == capi.CCT_ERR_INVALID and b"reserve_fusion" in lib.cct_last_error_string(ctx.h)
    f = capi.BwdFusion(None, None, None, 0, 0, 1)  # neither dY nor dP
    rc = lib.cct_conv_backward_fused(plan, vp(buf.ptr), vp(buf.ptr), None, C.byref(f), None, vp(buf.ptr), vp(buf.ptr))
    assert rc == capi.CCT_ERR_INVALID
    capi.check(lib.cct_conv_plan_destroy(plan), "destroy", ctx.h)
    buf.free()
