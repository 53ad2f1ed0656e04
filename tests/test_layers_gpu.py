"""GPU parity of the CaffeNet bridges around the contractions, through the C ABI: local response normalisation,
dropout, softmax with loss, max pooling forward on staged planes.  LRN and softmax are fp32 arithmetic with pow / exp /
log (tolerance 1e-4 max-norm, tests/parity.py) against the numpy restatements pinned to the reference's CPU bridges
(tests/test_layers_oracle.py) and, where oracle/_ref is present, against those bridges directly; dropout and pooling
are copy / compare work and must be bit-exact."""
import ctypes as C

import numpy as np
import pytest

from caffecontroll_b200 import capi
from caffecontroll_b200.bridge import LogicalCube
from oracle import pyoracle
from tests.parity import assert_close

pytestmark = pytest.mark.gpu
vp = C.c_void_p


@pytest.mark.parametrize("shape", [(3, 8, 5, 5), (4, 96, 27, 5), (2, 256, 13, 5), (2, 7, 6, 3), (2, 9, 4, 7)])
def test_lrn_forward_backward(ctx, shape):
    B, D, n, local = shape
    rng = np.random.default_rng(31 + D)
    X = np.maximum(rng.standard_normal((B, D, n, n), dtype=np.float32) * 8, 0)
    dY = rng.standard_normal((B, D, n, n), dtype=np.float32)
    alpha, beta = 1e-1, 0.75
    Yr, scale_r = pyoracle.np_lrn_forward(X, local, alpha, beta)
    dXr = pyoracle.np_lrn_backward(X, dY, local, alpha, beta)
    lib = ctx.lib
    cX, cdY = LogicalCube.from_numpy(ctx, X), LogicalCube.from_numpy(ctx, dY)
    cY, cS, cdX = (LogicalCube(ctx, n, n, D, B) for _ in range(3))
    capi.check(lib.cct_lrn_forward(ctx.h, vp(cX.ptr), vp(cY.ptr), vp(cS.ptr), B, D, n * n, local, alpha, beta), "lrn fwd", ctx.h)
    capi.check(lib.cct_lrn_backward(ctx.h, vp(cX.ptr), vp(cY.ptr), vp(cS.ptr), vp(cdY.ptr), vp(cdX.ptr), B, D, n * n, local,
                                    alpha, beta), "lrn bwd", ctx.h)
    ctx.sync()
    assert_close(cY.download(), Yr, "LRN Y")
    assert_close(cS.download(), scale_r, "LRN scale")
    assert_close(cdX.download(), dXr, "LRN dX")
    ref = pyoracle.reference()
    if ref is not None:
        Yb, dXb, _ = ref.lrn(X, local, alpha, beta, dY=dY)
        assert_close(cY.download(), Yb, "LRN Y vs the reference bridge")
        assert_close(cdX.download(), dXb, "LRN dX vs the reference bridge")
    # without the denominator cube: the forward pass does not store it, the backward pass forms it again from X
    cY2, cdX2 = LogicalCube(ctx, n, n, D, B), LogicalCube(ctx, n, n, D, B)
    capi.check(lib.cct_lrn_forward(ctx.h, vp(cX.ptr), vp(cY2.ptr), vp(None), B, D, n * n, local, alpha, beta), "lrn fwd", ctx.h)
    rc = lib.cct_lrn_backward(ctx.h, vp(cX.ptr), vp(None), vp(None), vp(cdY.ptr), vp(cdX2.ptr), B, D, n * n, local, alpha, beta)
    ctx.sync()
    assert np.array_equal(cY2.download(), cY.download())
    if local in (3, 5):
        capi.check(rc, "lrn bwd without scale", ctx.h)
        assert np.array_equal(cdX2.download(), cdX.download())
    else:
        assert rc == capi.CCT_ERR_UNSUPPORTED
    for c in (cX, cdY, cY, cS, cdX, cY2, cdX2):
        c.free()


def test_lrn_caffenet_parameters_are_not_the_identity(ctx):
    # alpha 1e-4, beta 0.75 on pool1-sized activations of realistic magnitude
    B, D, n = 2, 96, 27
    rng = np.random.default_rng(32)
    X = np.maximum(rng.standard_normal((B, D, n, n), dtype=np.float32) * 40, 0)
    Yr, _ = pyoracle.np_lrn_forward(X, 5, 1e-4, 0.75)
    assert np.max(np.abs(Yr - X)) > 1e-2 * np.max(X)
    cX = LogicalCube.from_numpy(ctx, X)
    cY, cS = LogicalCube(ctx, n, n, D, B), LogicalCube(ctx, n, n, D, B)
    capi.check(ctx.lib.cct_lrn_forward(ctx.h, vp(cX.ptr), vp(cY.ptr), vp(cS.ptr), B, D, n * n, 5, 1e-4, 0.75), "lrn", ctx.h)
    ctx.sync()
    assert_close(cY.download(), Yr, "LRN Y (CaffeNet parameters)")
    for c in (cX, cY, cS):
        c.free()


def test_dropout_apply_is_bit_exact(ctx):
    rng = np.random.default_rng(33)
    X = rng.standard_normal((6, 4096, 1, 1), dtype=np.float32)
    mask = (rng.random(X.shape) < 0.5).astype(np.uint32)
    ref = pyoracle.reference()
    if ref is not None:  # the mask the reference bridge draws from its own generator
        Yb, mask, _, _ = ref.dropout(X, 0.5, 11)
    cX, cM = LogicalCube.from_numpy(ctx, X), LogicalCube.from_numpy(ctx, mask)
    cY = LogicalCube(ctx, 1, 1, 4096, 6)
    capi.check(ctx.lib.cct_dropout_apply(ctx.h, vp(cX.ptr), vp(cM.ptr), 2.0, vp(cY.ptr), X.size), "dropout", ctx.h)
    ctx.sync()
    Y = cY.download()
    assert np.array_equal(Y, X * mask * np.float32(2.0))
    if ref is not None:
        assert np.array_equal(Y, Yb)
    for c in (cX, cM, cY):
        c.free()


def test_device_dropout_mask_is_reproducible_and_has_the_right_rate(ctx):
    n = 256 * 4096
    a, b, c = (LogicalCube(ctx, 1, 1, 4096, 256, np.uint32) for _ in range(3))
    lib = ctx.lib
    capi.check(lib.cct_dropout_mask(ctx.h, vp(a.ptr), n, 0.5, 7, 1), "mask", ctx.h)
    capi.check(lib.cct_dropout_mask(ctx.h, vp(b.ptr), n, 0.5, 7, 1), "mask", ctx.h)
    capi.check(lib.cct_dropout_mask(ctx.h, vp(c.ptr), n, 0.25, 7, 2), "mask", ctx.h)
    ctx.sync()
    ma, mb, mc = a.download(), b.download(), c.download()
    assert np.array_equal(ma, mb) and set(np.unique(ma)) == {0, 1}
    assert abs(ma.mean() - 0.5) < 0.005 and abs(mc.mean() - 0.75) < 0.005
    assert not np.array_equal(ma, mc)
    for x in (a, b, c):
        x.free()


@pytest.mark.parametrize("shape", [(16, 50), (256, 1000), (3, 7)])
def test_softmax_loss(ctx, shape):
    B, Cn = shape
    rng = np.random.default_rng(34 + Cn)
    X = (3 * rng.standard_normal((B, Cn, 1, 1))).astype(np.float32)
    labels = rng.integers(0, Cn, B).astype(np.float32)
    pr, lr, gr = pyoracle.np_softmax_loss(X, labels, scale=1.0 / (4 * B))  # a job four times this partition's batch
    cX, cL = LogicalCube.from_numpy(ctx, X), LogicalCube.from_numpy(ctx, labels.reshape(B, 1, 1, 1))
    cP, cG = LogicalCube(ctx, 1, 1, Cn, B), LogicalCube(ctx, 1, 1, Cn, B)
    cIL, cLoss = LogicalCube(ctx, 1, 1, 1, B), LogicalCube(ctx, 1, 1, 1, 1)
    lib = ctx.lib
    capi.check(lib.cct_softmax_loss_forward(ctx.h, vp(cX.ptr), vp(cL.ptr), vp(cP.ptr), vp(cIL.ptr), vp(cLoss.ptr), B, Cn),
               "softmax fwd", ctx.h)
    capi.check(lib.cct_softmax_loss_backward(ctx.h, vp(cP.ptr), vp(cL.ptr), vp(cG.ptr), B, Cn, 1.0 / (4 * B)), "softmax bwd",
               ctx.h)
    ctx.sync()
    assert_close(cP.download(), pr, "softmax probabilities")
    loss = float(cLoss.download().reshape(-1)[0])
    assert abs(loss - lr) <= 1e-4 * abs(lr)
    assert_close(cG.download(), gr, "softmax-loss gradient")
    ref = pyoracle.reference()
    if ref is not None:
        pb, lb, gb, _ = ref.softmax_loss(X, labels)
        assert_close(cP.download(), pb, "probabilities vs the reference bridge")
        assert abs(loss - lb) <= 1e-4 * abs(lb)
        assert_close(cG.download() * np.float32(4.0), gb, "gradient vs the reference bridge (its scale is 1 / batch)")
    for c in (cX, cL, cP, cG, cIL, cLoss):
        c.free()


@pytest.mark.parametrize("shape", [(4, 96, 55, 3, 2), (2, 256, 27, 3, 2), (2, 256, 13, 3, 2), (1, 3, 224, 2, 2)])
def test_maxpool_forward_full_planes_bit_exact(ctx, port, shape):
    B, D, n, k, s = shape
    m = (n - k) // s + 1
    rng = np.random.default_rng(35 + n)
    A = np.maximum(rng.standard_normal((B, D, n, n), dtype=np.float32), 0)  # ReLU output: many ties at zero
    Yr, idxr = port.maxpool_forward(A, k, s)
    cA = LogicalCube.from_numpy(ctx, A)
    cY, cI = LogicalCube(ctx, m, m, D, B), LogicalCube(ctx, m, m, D, B, np.int32)
    capi.check(ctx.lib.cct_maxpool_forward(ctx.h, vp(cA.ptr), vp(cY.ptr), vp(cI.ptr), B * D, n, k, s), "pool fwd", ctx.h)
    ctx.sync()
    assert np.array_equal(cY.download(), Yr)
    assert np.array_equal(cI.download(), idxr)
    for c in (cA, cY, cI):
        c.free()
