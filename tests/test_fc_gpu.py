"""FullyConnectedBridge on the GPU against the CPU oracle: the tensor-core plan (three GEMMs that read X, W and dY in
place, reductions split over CTAs) and the 1x1-convolution fallback, the fused ReLU / dropout switches, ragged sizes
(features that are not multiples of the 128 x 32 tiles, batches that are not multiples of 32), and the three CaffeNet
layers fc6 / fc7 / fc8 at batch 256.  The oracle is a float64 matrix product (the reference's FullyConnectedBridge is
three sgemm calls, src/bridges/FullyConnectedBridge_impl.hxx:201-215, 305-312; its compiled CPU code checks the
restatement in tests/test_layers_oracle.py)."""
import warnings

import numpy as np
import pytest

from caffecontroll_b200 import FullyConnectedBridge, Layer, LogicalCube, capi
from tests.parity import TOL, assert_close, maxnorm_rel

pytestmark = pytest.mark.gpu

# (B, D, n, num_output): ragged small cases, then fc6's input geometry (256 x 6 x 6) at reduced batch and width
# and batches around the 128-column accumulator tile of the forward pass and the data gradient (1, 130, 200 images)
SHAPES = [(4, 3, 5, 10), (8, 16, 4, 40), (16, 64, 3, 96), (32, 256, 6, 512), (5, 7, 2, 12), (40, 33, 4, 200),
          (1, 64, 2, 20), (130, 8, 2, 260), (200, 32, 2, 136)]


def _oracle(X, W, b, dY):
    B, o = dY.shape[0], W.shape[0]
    X2, W2, dY2 = X.reshape(B, -1).astype(np.float64), W.reshape(o, -1).astype(np.float64), dY.reshape(B, o).astype(np.float64)
    Y = X2 @ W2.T + (b.astype(np.float64) if b is not None else 0.0)
    dX = dY2 @ W2
    dW = dY2.T @ X2
    db = dY2.sum(axis=0)
    return (Y.astype(np.float32).reshape(B, o, 1, 1), dX.astype(np.float32).reshape(X.shape),
            dW.astype(np.float32).reshape(W.shape), db.astype(np.float32))


def _run(ctx, X, W, b, dY, algo, relu=False, mask=None, scale=1.0, in_relu=False, in_mask=None, in_scale=1.0):
    B, D, n, _ = X.shape
    o = W.shape[0]
    xin = Layer(LogicalCube.from_numpy(ctx, X), LogicalCube(ctx, n, n, D, B))
    out = Layer(LogicalCube(ctx, 1, 1, o, B), LogicalCube.from_numpy(ctx, dY))
    fc = FullyConnectedBridge(xin, out, b is not None, algo)
    fc.p_model_cube.upload(W)
    if b is not None:
        fc.p_bias_cube.upload(b)
    cubes = []
    fc.fuse_relu, fc.fuse_relu_backward = relu, in_relu
    if mask is not None:
        fc.dropout_mask, fc.dropout_scale = LogicalCube.from_numpy(ctx, mask), scale
        cubes.append(fc.dropout_mask)
    if in_mask is not None:
        fc.input_dropout_mask, fc.input_dropout_scale = LogicalCube.from_numpy(ctx, in_mask), in_scale
        cubes.append(fc.input_dropout_mask)
    fc.forward()
    fc.backward()
    ctx.sync()
    res = (out.p_data_cube.download(), xin.p_gradient_cube.download(), fc.p_model_gradient_cube.download().reshape(W.shape),
           fc.p_bias_gradient_cube.download().reshape(-1) if b is not None else None, fc.algo)
    fc.close()
    for layer in (xin, out):
        layer.p_data_cube.free()
        layer.p_gradient_cube.free()
    for c in cubes:
        c.free()
    return res


@pytest.mark.parametrize("algo", [capi.ALGO_SIMT_FP32, capi.ALGO_UMMA_3XTF32, capi.ALGO_AUTO])
@pytest.mark.parametrize("shape", SHAPES)
def test_fully_connected_matches_oracle(ctx, shape, algo):
    B, D, n, o = shape
    K = D * n * n
    if algo == capi.ALGO_SIMT_FP32 and K * o > 200000:
        pytest.skip("the direct fp32 kernels are the small-shape fallback")
    if algo == capi.ALGO_UMMA_3XTF32 and (K % 4 or o % 4):
        pytest.skip("the tensor-core plan needs feature counts that are multiples of 4")
    rng = np.random.default_rng(77 + o)
    X = np.maximum(rng.standard_normal((B, D, n, n), dtype=np.float32), 0)
    W = (0.01 * rng.standard_normal((o, D, n, n))).astype(np.float32)
    b = (0.1 * rng.standard_normal(o)).astype(np.float32)
    dY = rng.standard_normal((B, o, 1, 1), dtype=np.float32)
    Yr, dXr, dWr, dbr = _oracle(X, W, b, dY)
    Y, dX, dW, db, used = _run(ctx, X, W, b, dY, algo)
    if algo != capi.ALGO_AUTO:
        assert used == algo
    for a, r, name in ((Y, Yr, "Y"), (dX, dXr, "dX"), (dW, dWr, "dW"), (db, dbr, "db")):
        assert_close(a, r, name)


def test_fused_relu_and_dropout_switches(ctx):
    B, D, n, o = 24, 16, 4, 64
    rng = np.random.default_rng(5)
    mask_in = (rng.random((B, D, n, n)) < 0.5).astype(np.uint32)
    X = (np.maximum(rng.standard_normal((B, D, n, n), dtype=np.float32), 0) * mask_in * 2.0).astype(np.float32)
    W = (0.05 * rng.standard_normal((o, D, n, n))).astype(np.float32)
    b = (0.1 * rng.standard_normal(o)).astype(np.float32)
    dY = rng.standard_normal((B, o, 1, 1), dtype=np.float32)
    mask_out = (rng.random((B, o, 1, 1)) < 0.5).astype(np.uint32)
    Yr, dXr, dWr, dbr = _oracle(X, W, b, dY)
    Y, dX, dW, db, _ = _run(ctx, X, W, b, dY, capi.ALGO_UMMA_3XTF32, relu=True, mask=mask_out, scale=2.0, in_relu=True,
                            in_mask=mask_in, in_scale=2.0)
    assert_close(Y, np.maximum(Yr, 0) * mask_out * np.float32(2.0), "Y with ReLU and dropout")
    want_dX = dXr * mask_in * np.float32(2.0) * (X > 0)
    assert_close(dX, want_dX.astype(np.float32), "dX with the dropout and ReLU bridges in front folded in")
    assert np.all(dX[(X <= 0) | (mask_in == 0)] == 0.0)
    assert_close(dW, dWr, "dW")
    assert_close(db, dbr, "db")


@pytest.mark.parametrize("layer", [("fc6", 256, 6, 4096), ("fc7", 4096, 1, 4096), ("fc8", 4096, 1, 1000)],
                         ids=["fc6", "fc7", "fc8"])
def test_caffenet_fc_layers_batch256(ctx, layer):
    name, D, n, o = layer
    B = 256
    rng = np.random.default_rng(900 + o + n)
    X = np.maximum(rng.standard_normal((B, D, n, n), dtype=np.float32), 0)
    W = (0.01 * rng.standard_normal((o, D, n, n))).astype(np.float32)
    b = np.ones(o, np.float32)
    dY = rng.standard_normal((B, o, 1, 1), dtype=np.float32)
    Yr, dXr, dWr, dbr = _oracle(X, W, b, dY)
    Y, dX, dW, db, used = _run(ctx, X, W, b, dY, capi.ALGO_AUTO)
    assert used == capi.ALGO_UMMA_3XTF32
    errs = {t: maxnorm_rel(a, r) for t, a, r in (("Y", Y, Yr), ("dX", dX, dXr), ("dW", dW, dWr), ("db", db, dbr))}
    warnings.warn("parity %s, batch 256: %s" % (name, ", ".join("%s %.2e" % kv for kv in errs.items())))
    for a, r, t in ((Y, Yr, "Y"), (dX, dXr, "dX"), (dW, dWr, "dW"), (db, dbr, "db")):
        assert_close(a, r, "%s %s" % (name, t))
