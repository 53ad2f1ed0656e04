"""GPU parity tests of the convolution bridge, called through the C ABI (caffecontroll_b200.bridge -> ctypes ->
libcct_b200.so) and checked against the CPU oracle on the same seeded inputs.

Tolerance (fp32 path): max-norm relative error <= 1e-4 per tensor plus the element-wise check with an rms floor
(tests/parity.py).  The oracle is the reference's compiled CPU code when oracle/_ref is present, else the plain-C
restatement; both are test infrastructure.
"""
import os

import numpy as np
import pytest

from tests.parity import TOL, assert_close, make_inputs, maxnorm_rel

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "conv_golden.npz")

SIMT, UMMA = 1, 2

# B, D, n, o, k, s, p, g
SHAPES = [
    (4, 3, 20, 10, 5, 4, 2, 1),     # the reference's fixture shape
    (2, 1, 28, 20, 5, 1, 0, 1),     # LeNet conv1 (batch reduced)
    (2, 3, 35, 8, 11, 4, 0, 1),     # 11x11 stride 4
    (2, 8, 9, 12, 5, 1, 2, 2),      # grouped 5x5 pad 2
    (3, 6, 7, 10, 3, 1, 1, 1),      # 3x3 pad 1
    (2, 4, 11, 6, 3, 2, 1, 1),      # stride 2
    (1, 2, 5, 3, 1, 1, 0, 1),       # 1x1
    (2, 4, 9, 4, 3, 3, 0, 2),       # stride == kernel, grouped
    (3, 4, 6, 9, 6, 1, 0, 1),       # kernel == input: a fully connected layer
    (1, 1, 3, 1, 3, 1, 1, 1),       # single channel, single filter
    (2, 5, 13, 7, 3, 5, 1, 1),      # stride larger than kernel: some input pixels receive no gradient
    (5, 48, 13, 40, 5, 1, 2, 1),    # K = 1200 like CaffeNet conv2, ragged pixel tile (845 pixels)
    (2, 16, 13, 272, 3, 1, 1, 1),   # 272 filters: two output-channel tiles of 136
    (2, 288, 6, 16, 3, 1, 1, 1),    # 288 input channels: two input-channel tiles in the data gradient
    (2, 128, 10, 136, 3, 2, 1, 2),  # 576 lowered rows per group, stride 2, pad 1: weight gradient through the gather kernel
    (2, 64, 8, 160, 3, 1, 1, 1),    # 160 filters in one tile: the one-CTA-per-SM shape, in all three passes
    (3, 10, 12, 100, 6, 1, 2, 1),   # 360 lowered rows, 100 filters, pad 2: weight gradient with dY through tensor memory
    (2, 24, 9, 48, 5, 1, 2, 2),     # the same kernel on a grouped layer (300 rows and 24 filters per group)
]


def _oracle(port, reference_or_none, X, W, b, dY, k, s, p, g, needs_dx=True):
    if reference_or_none is not None:
        Y, dX, dW, db = reference_or_none.conv_fwd_bwd(X, W, b, dY, k, s, p, g=g, partitions=1, needs_dx=needs_dx)
        return Y, dX, dW, db
    Y = port.conv_forward(X, W, b, k, s, p, g)
    dX, dW, db = port.conv_backward(X, W, dY, k, s, p, g, needs_dx=needs_dx, bias=b is not None)
    return Y, dX, dW, db


@pytest.fixture(scope="module")
def ref_or_none():
    from oracle import pyoracle
    return pyoracle.reference()


@pytest.mark.parametrize("algo", [SIMT, UMMA])
@pytest.mark.parametrize("shape", SHAPES)
def test_conv_fwd_bwd_matches_oracle(ctx, port, ref_or_none, shape, algo):
    from caffecontroll_b200 import conv_layer
    B, D, n, o, k, s, p, g = shape
    X, W, b, dY = make_inputs(11, B, D, n, o, k, s, p, g)
    Yr, dXr, dWr, dbr = _oracle(port, ref_or_none, X, W, b, dY, k, s, p, g)
    Y, dX, dW, db, used = conv_layer(ctx, X, W, b, dY, k, s, p, g, algo=algo)
    assert used == algo
    for a, r, name in ((Y, Yr, "Y"), (dX, dXr, "dX"), (dW, dWr, "dW"), (db, dbr, "db")):
        assert_close(a, r, name)


@pytest.mark.parametrize("algo", [SIMT, UMMA])
def test_committed_reference_fixtures(ctx, algo):
    from caffecontroll_b200 import conv_layer
    z = np.load(GOLDEN)
    for name in sorted({k.split("/")[0] for k in z.files if k.endswith("/dW")}):
        B, D, n, o, k, s, p, g = (int(v) for v in z[name + "/shape"])
        Y, dX, dW, db, _ = conv_layer(ctx, z[name + "/X"], z[name + "/W"], z[name + "/b"], z[name + "/dY"], k, s, p, g,
                                      algo=algo)
        for a, t in ((Y, "Y"), (dX, "dX"), (dW, "dW"), (db, "db")):
            assert_close(a, z[name + "/" + t], "%s/%s" % (name, t))


@pytest.mark.parametrize("algo", [SIMT, UMMA])
def test_no_bias_no_dx_and_fused_relu(ctx, port, algo):
    from caffecontroll_b200 import conv_layer
    B, D, n, o, k, s, p, g = 3, 6, 12, 10, 3, 1, 1, 1
    X, W, b, dY = make_inputs(12, B, D, n, o, k, s, p, g)
    Y, dX, dW, db, _ = conv_layer(ctx, X, W, None, dY, k, s, p, g, needs_dx=False, algo=algo)
    assert dX is None and db is None
    assert_close(Y, port.conv_forward(X, W, None, k, s, p, g), "Y without bias")
    _, dWr, _ = port.conv_backward(X, W, dY, k, s, p, g, needs_dx=False, bias=False)
    assert_close(dW, dWr, "dW without dX")
    Yrelu = conv_layer(ctx, X, W, b, None, k, s, p, g, algo=algo, relu=True)[0]
    assert_close(Yrelu, port.relu_forward(port.conv_forward(X, W, b, k, s, p, g)), "fused ReLU")


def test_umma_and_simt_agree_on_lenet_conv1_full_batch(ctx, port):
    # BASELINE config 1 at full size: 64x1x28x28 ~U(0,1), 20 filters 5x5; the oracle finishes in well under a second.
    from caffecontroll_b200 import conv_layer
    X, W, b, dY = make_inputs(1000, 64, 1, 28, 20, 5, 1, 0, x_dist="uniform")
    Yr = port.conv_forward(X, W, b, 5, 1, 0)
    dXr, dWr, dbr = port.conv_backward(X, W, dY, 5, 1, 0)
    for algo in (SIMT, UMMA):
        Y, dX, dW, db, _ = conv_layer(ctx, X, W, b, dY, 5, 1, 0, algo=algo)
        for a, r, name in ((Y, Yr, "Y"), (dX, dXr, "dX"), (dW, dWr, "dW"), (db, dbr, "db")):
            assert_close(a, r, name)


def test_linearity_and_adjoint_at_larger_size(ctx):
    """Size-independent properties on a CaffeNet conv3-like layer (no oracle run):
    conv(a*X1 + X2) = a*conv(X1) + conv(X2) (bias off), and <conv(X), dY> = <X, dgrad(dY)> = <W, wgrad(X, dY)>."""
    from caffecontroll_b200 import conv_layer
    B, D, n, o, k, s, p, g = 8, 64, 13, 96, 3, 1, 1, 1
    X1, W, _, dY = make_inputs(13, B, D, n, o, k, s, p, g)
    X2 = make_inputs(14, B, D, n, o, k, s, p, g)[0]
    Y1, dX, dW, _, _ = conv_layer(ctx, X1, W, None, dY, k, s, p, g, algo=UMMA)
    Y2 = conv_layer(ctx, X2, W, None, None, k, s, p, g, algo=UMMA)[0]
    Y12 = conv_layer(ctx, (np.float32(0.5) * X1 + X2), W, None, None, k, s, p, g, algo=UMMA)[0]
    assert maxnorm_rel(Y12, np.float32(0.5) * Y1 + Y2) <= TOL
    lhs = float(np.sum(Y1.astype(np.float64) * dY))
    assert abs(lhs - float(np.sum(X1.astype(np.float64) * dX))) <= TOL * abs(lhs) + 1e-3
    assert abs(lhs - float(np.sum(W.astype(np.float64) * dW))) <= TOL * abs(lhs) + 1e-3


@pytest.mark.parametrize("cfg", [
    ("AlexNet conv1 (BASELINE config 2)", 256, 3, 227, 96, 11, 4, 0, 1, "normal"),
    ("CaffeNet conv2 (BASELINE config 3)", 256, 96, 27, 256, 5, 1, 2, 2, "relu"),
])
def test_full_size_configs_by_properties(ctx, port, cfg):
    """The BASELINE layers at their full batch, where the CPU oracle would take minutes: images are independent in
    Y and dX, so the first and last image are compared with the oracle run on those two images alone; dW and db couple
    the whole batch and are pinned by the adjoint identity <conv(X), dY> = <X, dX> = <W, dW> (bias off in the
    identity's forward) and by db = plane sums of dY in float64."""
    from caffecontroll_b200 import conv_layer
    name, B, D, n, o, k, s, p, g, dist = cfg
    X, W, b, dY = make_inputs(2000 + n, B, D, n, o, k, s, p, g, relu_input=(dist == "relu"))
    Y, dX, dW, db, _ = conv_layer(ctx, X, W, b, dY, k, s, p, g, algo=UMMA)
    ends = [0, B - 1]
    Xe, dYe = np.ascontiguousarray(X[ends]), np.ascontiguousarray(dY[ends])
    Yr = port.conv_forward(Xe, W, b, k, s, p, g)
    dXr, _, _ = port.conv_backward(Xe, W, dYe, k, s, p, g)
    assert_close(Y[ends], Yr, name + ": Y of the first and last image")
    assert_close(dX[ends], dXr, name + ": dX of the first and last image")
    Y0 = Y - b.reshape(1, o, 1, 1)  # forward without bias, for the identity
    lhs = float(np.sum(Y0.astype(np.float64) * dY))
    assert abs(lhs - float(np.sum(X.astype(np.float64) * dX))) <= TOL * abs(lhs) + 1e-2
    assert abs(lhs - float(np.sum(W.astype(np.float64) * dW.reshape(W.shape)))) <= TOL * abs(lhs) + 1e-2
    db_ref = dY.astype(np.float64).sum(axis=(0, 2, 3))
    assert maxnorm_rel(db.reshape(-1), db_ref.astype(np.float32)) <= TOL


def test_backward_is_deterministic(ctx):
    from caffecontroll_b200 import conv_layer
    X, W, b, dY = make_inputs(15, 6, 16, 14, 24, 3, 1, 1, 1)
    a = conv_layer(ctx, X, W, b, dY, 3, 1, 1, algo=UMMA)
    c = conv_layer(ctx, X, W, b, dY, 3, 1, 1, algo=UMMA)
    for u, v in zip(a[:4], c[:4]):
        assert np.array_equal(u, v)


@pytest.mark.parametrize("B", [4, 20, 16])  # 4: one piece; 20 and 16: pipelined in slices of 3 (last one short) and 2
def test_host_buffer_entry_points(ctx, port, B):
    import ctypes as C
    from caffecontroll_b200 import capi
    D, n, o, k, s, p, g = 3, 20, 10, 5, 4, 2, 1
    X, W, b, dY = make_inputs(16, B, D, n, o, k, s, p, g)
    lib = ctx.lib
    desc = capi.ConvDesc(B, D, n, o, k, s, p, g, 1, capi.ALGO_AUTO)
    plan = C.c_void_p()
    capi.check(lib.cct_conv_plan_create(ctx.h, C.byref(desc), C.byref(plan)), "plan", ctx.h)
    Y = np.empty((B, o, 5, 5), np.float32)
    dX, dW, db = np.empty_like(X), np.empty_like(W), np.empty_like(b)
    vp = lambda a: a.ctypes.data_as(C.c_void_p)
    Yr = port.conv_forward(X, W, b, k, s, p, g)
    dXr, dWr, dbr = port.conv_backward(X, W, dY, k, s, p, g)
    for rnd in range(2):  # the second round reuses the staged X / W (NULL) and must not be disturbed by the first
        Y.fill(np.nan); dX.fill(np.nan); dW.fill(np.nan); db.fill(np.nan)
        capi.check(lib.cct_conv_forward_host(plan, vp(X), vp(W), vp(b), vp(Y), 0), "forward_host", ctx.h)
        if rnd == 0:
            capi.check(lib.cct_conv_backward_host(plan, vp(X), vp(W), vp(dY), vp(dX), vp(dW), vp(db)), "backward_host", ctx.h)
        else:
            capi.check(lib.cct_conv_backward_host(plan, None, None, vp(dY), vp(dX), vp(dW), vp(db)), "backward_host", ctx.h)
        assert_close(Y, Yr, "Y")
        for a, r, name in ((dX, dXr, "dX"), (dW, dWr, "dW"), (db, dbr, "db")):
            assert_close(a, r, name)
    # without dX
    dW.fill(np.nan)
    capi.check(lib.cct_conv_backward_host(plan, None, None, vp(dY), None, vp(dW), vp(db)), "backward_host", ctx.h)
    assert_close(dW, dWr, "dW without dX")
    lib.cct_conv_plan_destroy(plan)
