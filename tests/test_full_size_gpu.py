"""GPU parity at the BASELINE sizes: every CaffeNet convolution layer at batch 256 (configs 2 and 3 among them),
element-wise Y, dX, dW, db against the reference's own compiled CPU bridges (oracle/_ref: ParallelizedBridge over
ConvolutionBridge with the partition count DeepNet would use), and config 3's fused backward against the reference's
MaxPoolingBridge -> ReLUBridge -> ConvolutionBridge chain at batch 256.

Tolerance: max-norm relative error <= 1e-4 per tensor plus the element-wise check with an rms floor (tests/parity.py).
The four errors of every case are emitted as warnings so that they show in the summary of a quiet pytest run.
"""
import ctypes as C
import warnings

import numpy as np
import pytest

from tests.parity import assert_close, make_inputs, maxnorm_rel

pytestmark = pytest.mark.gpu

UMMA = 2
# name, B, D, n, o, k, s, p, g, input distribution
LAYERS = [
    ("AlexNet conv1 (BASELINE config 2)", 256, 3, 227, 96, 11, 4, 0, 1, "normal"),
    ("CaffeNet conv2 (BASELINE config 3)", 256, 96, 27, 256, 5, 1, 2, 2, "relu"),
    ("CaffeNet conv3", 256, 256, 13, 384, 3, 1, 1, 1, "relu"),
    ("CaffeNet conv4", 256, 384, 13, 384, 3, 1, 1, 2, "relu"),
    ("CaffeNet conv5", 256, 384, 13, 256, 3, 1, 1, 2, "relu"),
]


def _report(name, pairs):
    errs = {t: maxnorm_rel(a, r) for t, a, r in pairs}
    warnings.warn("parity %s: %s" % (name, ", ".join("%s %.2e" % (t, e) for t, e in errs.items())))
    for t, a, r in pairs:
        assert_close(a, r, "%s: %s" % (name, t))


@pytest.mark.parametrize("layer", LAYERS, ids=[l[0].split(" (")[0].replace(" ", "_") for l in LAYERS])
def test_caffenet_layers_batch256_elementwise_vs_reference(ctx, reference, layer):
    from caffecontroll_b200 import conv_layer
    name, B, D, n, o, k, s, p, g, dist = layer
    X, W, b, dY = make_inputs(3000 + n + o, B, D, n, o, k, s, p, g, relu_input=(dist == "relu"))
    parts = reference.default_partitions(B)
    Yr, dXr, dWr, dbr = reference.conv_fwd_bwd(X, W, b, dY, k, s, p, g=g, partitions=parts)
    Y, dX, dW, db, used = conv_layer(ctx, X, W, b, dY, k, s, p, g, algo=UMMA)
    assert used == UMMA
    _report(name + ", batch 256", (("Y", Y, Yr), ("dX", dX, dXr), ("dW", dW, dWr), ("db", db, dbr)))


def test_config3_fused_backward_batch256_vs_reference_bridges(ctx, reference):
    """conv2 -> ReLU -> 3x3/2 max-pool at batch 256: the pooled gradient goes through cct_conv_backward_fused (output
    gradient rebuilt from the pooling indices and the ReLU sign, input gradient masked by the ReLU in front) and
    through the reference's three bridges.  The reference chain starts from the forward output the device produced
    (checked against the reference's own forward first): started from its own forward, a 1e-6 difference could flip
    the winner of a near-tie inside a pooling window."""
    from caffecontroll_b200 import capi
    from caffecontroll_b200.bridge import LogicalCube
    B, D, n, o, k, s, p, g, pk, ps = 256, 96, 27, 256, 5, 1, 2, 2, 3, 2
    m = (n + 2 * p - k) // s + 1
    mp = (m - pk) // ps + 1
    X, W, _, _ = make_inputs(3333, B, D, n, o, k, s, p, g, relu_input=True)
    bias = np.ones(o, np.float32)  # CaffeNet conv2's bias filler
    dP = np.random.default_rng(3334).standard_normal((B, o, mp, mp), dtype=np.float32)
    lib, vp = ctx.lib, C.c_void_p
    desc = capi.ConvDesc(B, D, n, o, k, s, p, g, 1, UMMA)
    plan = C.c_void_p()
    capi.check(lib.cct_conv_plan_create(ctx.h, C.byref(desc), C.byref(plan)), "plan", ctx.h)
    capi.check(lib.cct_conv_plan_reserve_fusion(plan), "reserve", ctx.h)
    cX, cW, cb, cdP = (LogicalCube.from_numpy(ctx, a) for a in (X, W, bias, dP))
    cY, cPool = LogicalCube(ctx, m, m, o, B), LogicalCube(ctx, mp, mp, o, B)
    cidx = LogicalCube(ctx, mp, mp, o, B, np.int32)
    cdX, cdW, cdb = LogicalCube(ctx, n, n, D, B), LogicalCube(ctx, k, k, D // g, o), LogicalCube(ctx, 1, 1, o, 1)
    capi.check(lib.cct_conv_forward(plan, vp(cX.ptr), vp(cW.ptr), vp(cb.ptr), vp(cY.ptr), 1), "fwd", ctx.h)
    capi.check(lib.cct_maxpool_forward(ctx.h, vp(cY.ptr), vp(cPool.ptr), vp(cidx.ptr), B * o, m, pk, ps), "pool", ctx.h)
    f = capi.BwdFusion(cY.ptr, cidx.ptr, cdP.ptr, pk, ps, 1)
    capi.check(lib.cct_conv_backward_fused(plan, vp(cX.ptr), vp(cW.ptr), None, C.byref(f), vp(cdX.ptr), vp(cdW.ptr),
                                           vp(cdb.ptr)), "bwd fused", ctx.h)
    ctx.sync()
    A, P, idx = cY.download(), cPool.download(), cidx.download()
    dX, dW, db = cdX.download(), cdW.download(), cdb.download().reshape(-1)
    capi.check(lib.cct_conv_plan_destroy(plan), "destroy", ctx.h)
    for c in (cX, cW, cb, cdP, cY, cPool, cidx, cdX, cdW, cdb):
        c.free()

    parts = reference.default_partitions(B)
    # forward: convolution bridge then ReLU bridge
    zero_dY = np.zeros((B, o, m, m), np.float32)
    Yr = reference.conv_fwd_bwd(X, W, bias, zero_dY, k, s, p, g=g, partitions=parts, needs_dx=False)[0]
    Ar, _ = reference.relu(Yr)
    assert_close(A, Ar, "conv2 + ReLU forward")
    # backward chain from the device's forward output
    Pr, idxr, dAr = reference.maxpool(A, pk, ps, dY=dP)
    assert np.array_equal(P, Pr) and np.array_equal(idx, idxr)
    _, dYr = reference.relu(A, dY=dAr)  # A > 0 exactly where the pre-ReLU output was
    _, dXr, dWr, dbr = reference.conv_fwd_bwd(X, W, bias, dYr, k, s, p, g=g, partitions=parts)
    _, dXr = reference.relu(X, dY=dXr)  # the ReLU bridge in front of conv2
    _report("config 3 fused backward, batch 256", (("dX", dX, dXr), ("dW", dW, dWr), ("db", db, dbr)))
    assert np.all(dX[X <= 0] == 0.0)
