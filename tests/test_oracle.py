"""CPU tests (no GPU): pin the plain-C restatement (oracle/conv_oracle.c) against
  (1) the reference's own golden files, read in place when the reference tree is mounted,
  (2) the reference's compiled CPU code (oracle/_ref) on seeded inputs,
  (3) the committed fixtures generated from that code (tests/golden/conv_golden.npz),
and check the algebraic properties the parity tests rely on at sizes where no oracle is run.
"""
import os

import numpy as np
import pytest

from oracle.build import reference_root
from tests.parity import assert_close, make_inputs, maxnorm_rel

REF_TESTS = os.path.join(reference_root(), "tests")
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "conv_golden.npz")
needs_ref_tree = pytest.mark.skipif(not os.path.isdir(REF_TESTS), reason="reference tree not mounted")


def _load(rel):
    with open(os.path.join(REF_TESTS, rel)) as f:
        return np.array(f.read().split(), dtype=np.float32)


@needs_ref_tree
def test_port_reproduces_reference_small_fixtures(port):
    # tests/test_parallelized_convolution.cpp:123-270 of the reference: B=4, D=3, 20x20, 10 filters 5x5 s4 p2,
    # dY[i] = 0.1*i, SGD lr 0.01 without momentum; tolerance there is EPS = 1e-3 absolute.
    B, D, n, o, k, s, p, m = 4, 3, 20, 10, 5, 4, 2, 5
    X = _load("input/conv_forward_in.txt").reshape(B, D, n, n)
    b = _load("input/conv_bias_in.txt")
    Y = port.conv_forward(X, _load("input/conv_model.txt").reshape(o, D, k, k), b, k, s, p)
    Yg = _load("output/conv_forward.txt").reshape(B, o, m, m)
    assert np.max(np.abs(Y - Yg)) <= 1e-3
    W = _load("input/conv_backward_model.txt").reshape(o, D, k, k)
    dY = np.array([0.1 * i for i in range(B * o * m * m)], np.float32).reshape(B, o, m, m)
    dX, dW, db = port.conv_backward(X, W, dY, k, s, p)
    assert np.max(np.abs(dX.ravel() - _load("output/conv_backward.txt"))) <= 1e-3
    assert np.max(np.abs((b - np.float32(0.01) * db) - _load("output/conv_bias.txt"))) <= 1e-3
    assert np.max(np.abs((W - np.float32(0.01) * dW).ravel() - _load("output/conv_weights.txt"))) <= 1e-3


@needs_ref_tree
def test_port_reproduces_reference_large_fixtures(port):
    # tests/test_parallelized_convolution_large_CPU.cpp: B=4, D=3, 127x127, 8 filters 11x11 s4 p2 (m=31);
    # tolerance max(0.01, 1%) (:149,223,244,267).  The dX file holds only the first 30752 values (:208-216).
    B, D, n, o, k, s, p, m = 4, 3, 127, 8, 11, 4, 2, 31
    X = _load("input/conv_forward_in_large.txt").reshape(B, D, n, n)
    W = _load("input/conv_model_large.txt").reshape(o, D, k, k)
    b = _load("input/conv_bias_in_large.txt")
    Y = port.conv_forward(X, W, b, k, s, p)
    Yg = _load("output/conv_forward_large.txt")
    assert Yg.size == B * o * m * m

    def close(a, g):
        return np.all(np.abs(a - g) <= np.maximum(0.01, 0.01 * np.abs(g)))

    assert close(Y.ravel(), Yg)
    Wb = _load("input/conv_backward_model_large.txt").reshape(o, D, k, k)
    dY = np.array([0.1 * i for i in range(B * o * m * m)], np.float32).reshape(B, o, m, m)
    dX, dW, db = port.conv_backward(X, Wb, dY, k, s, p)
    dXg = _load("output/conv_backward_large.txt")
    assert close(dX.ravel()[:dXg.size], dXg)
    assert close(b - np.float32(0.01) * db, _load("output/conv_bias_large.txt"))
    assert close((Wb - np.float32(0.01) * dW).ravel(), _load("output/conv_weights_large.txt"))


@needs_ref_tree
def test_port_masks_reproduce_reference_fixtures(port):
    # tests/test_MaxPooling_bridge.cpp (B=5, D=3, 10x10, k=4, s=2, dY = i) and tests/test_ReLU_bridge.cpp (5x3x20x20).
    A = _load("input/pooling_forward_in.txt").reshape(5, 3, 10, 10)
    Y, idx = port.maxpool_forward(A, 4, 2)
    assert np.max(np.abs(Y.ravel() - _load("output/pooling_forward.txt"))) <= 1e-3
    dY = np.arange(Y.size, dtype=np.float32).reshape(Y.shape)
    dA = port.maxpool_backward(dY, idx, 10)
    assert np.max(np.abs(dA.ravel() - _load("output/pooling_backward.txt"))) <= 1e-3
    R = _load("input/relu_forward_in.txt")
    assert np.max(np.abs(port.relu_forward(R) - _load("output/relu_forward.txt"))) <= 1e-3
    gold = _load("output/relu_backward.txt")
    dR = port.relu_backward(R, np.arange(R.size, dtype=np.float32))
    if np.max(np.abs(dR - gold)) > 1e-3:  # the reference test may use another upstream gradient; the mask must agree
        assert np.array_equal(dR != 0, (gold != 0) | (np.arange(R.size) == 0))


CASES = [  # B, D, n, o, k, s, p, g
    (4, 3, 20, 10, 5, 4, 2, 1), (2, 1, 28, 20, 5, 1, 0, 1), (2, 3, 35, 8, 11, 4, 0, 1), (2, 8, 9, 12, 5, 1, 2, 2),
    (3, 6, 7, 10, 3, 1, 1, 1), (2, 4, 11, 6, 3, 2, 1, 1), (1, 2, 5, 3, 1, 1, 0, 1), (2, 4, 9, 4, 3, 3, 0, 2),
]


@pytest.mark.parametrize("case", CASES)
def test_port_matches_compiled_reference(port, reference, case):
    B, D, n, o, k, s, p, g = case
    X, W, b, dY = make_inputs(7, B, D, n, o, k, s, p, g)
    Yr, dXr, dWr, dbr = reference.conv_fwd_bwd(X, W, b, dY, k, s, p, g=g, partitions=min(2, B))
    Y = port.conv_forward(X, W, b, k, s, p, g)
    dX, dW, db = port.conv_backward(X, W, dY, k, s, p, g)
    for a, r, name in ((Y, Yr, "Y"), (dX, dXr, "dX"), (dW, dWr, "dW"), (db, dbr, "db")):
        assert_close(a, r, name, tol=2e-6 * max(1, k * k * D // g) ** 0.5 + 1e-5)


def test_port_matches_committed_reference_fixtures(port):
    z = np.load(GOLDEN)
    names = sorted({k.split("/")[0] for k in z.files if k.endswith("/dW")})
    assert len(names) >= 7
    for name in names:
        B, D, n, o, k, s, p, g = (int(v) for v in z[name + "/shape"])
        X, W, b, dY = (z[name + "/" + t] for t in ("X", "W", "b", "dY"))
        Y = port.conv_forward(X, W, b, k, s, p, g)
        dX, dW, db = port.conv_backward(X, W, dY, k, s, p, g)
        for a, t in ((Y, "Y"), (dX, "dX"), (dW, "dW"), (db, "db")):
            assert_close(a, z[name + "/" + t], name + "/" + t, tol=2e-5)
    for name in ("pool3s2", "pool4s2"):
        B, D, n, k, s = (int(v) for v in z[name + "/shape"])
        Y, idx = port.maxpool_forward(z[name + "/A"], k, s)
        assert np.array_equal(Y, z[name + "/Y"]) and np.array_equal(idx, z[name + "/idx"])
        dA = port.maxpool_backward(z[name + "/dP"], idx, n)
        assert np.array_equal(dA, z[name + "/dA_pool"])
        assert np.array_equal(port.relu_backward(z[name + "/A"], dA), z[name + "/dA_pool_relu"])


def test_sgd_two_steps_matches_reference_fixture(port):
    # SGDGradientUpdater with momentum 0.9 and L2 decay 0.0005 applied twice by the reference bridge.
    z = np.load(GOLDEN)
    name = "ref_small_fixture_shape"
    B, D, n, o, k, s, p, g = (int(v) for v in z[name + "/shape"])
    X, W, b, dY = (z[name + "/" + t].copy() for t in ("X", "W", "b", "dY"))
    hw, hb = np.zeros_like(W), np.zeros_like(b)
    for it in (1, 2):
        _, dW, db = port.conv_backward(X, W, dY, k, s, p, g)
        lr = port.learning_rate("step", 0.01, 0.1, float(it), 100000.0)
        port.sgd_update(W, dW, hw, lr, 0.9, 0.0005)
        port.sgd_update(b, db, hb, lr, 0.9, 0.0005)
    assert_close(W, z["sgd_two_steps/W"], "W after 2 SGD steps", tol=1e-5)
    assert_close(b, z["sgd_two_steps/b"], "bias after 2 SGD steps", tol=1e-5)


def test_lowering_matches_sliding_window(port):
    # tests/test_connector.cpp:18-42 of the reference checks lower_cube against an in-test restatement of eq. 4.
    rng = np.random.default_rng(3)
    for (B, D, n, k, s, p) in ((2, 3, 4, 2, 1, 0), (1, 2, 7, 3, 2, 1), (2, 1, 6, 5, 1, 2)):
        X = rng.standard_normal((B, D, n, n), dtype=np.float32)
        m = (n + 2 * p - k) // s + 1
        Xp = np.pad(X, ((0, 0), (0, 0), (p, p), (p, p)))
        want = np.empty((B, m, m, D, k, k), np.float32)
        for r in range(m):
            for c in range(m):
                want[:, r, c] = Xp[:, :, r * s:r * s + k, c * s:c * s + k]
        assert np.array_equal(port.lower(X, k, s, p), want.reshape(B * m * m, D * k * k))


def test_inverse_lowering_is_adjoint_of_lowering(port):
    # <lower(X), G^T> == <X, inverse_lower(G)>: the only pin the reference has on inverse_lower_cube is dX itself.
    rng = np.random.default_rng(4)
    for (B, D, n, k, s, p) in ((2, 3, 9, 3, 2, 1), (1, 2, 11, 5, 1, 2), (2, 2, 12, 4, 4, 0)):
        m = (n + 2 * p - k) // s + 1
        X = rng.standard_normal((B, D, n, n), dtype=np.float32)
        G = rng.standard_normal((D * k * k, B * m * m), dtype=np.float32)
        lhs = np.sum(port.lower(X, k, s, p).astype(np.float64) * G.T.astype(np.float64))
        rhs = np.sum(X.astype(np.float64) * port.inverse_lower(G, B, D, n, k, s, p).astype(np.float64))
        assert abs(lhs - rhs) <= 1e-5 * max(1.0, abs(lhs))


def test_full_size_kernel_equals_fully_connected(port):
    # Metamorphic pin used by the reference (tests/test_fc_bridge.cpp:89-98,222-231): conv with k = n is an FC layer.
    X, W, b, dY = make_inputs(5, 7, 12, 6, 25, 6, 1, 0)
    Y = port.conv_forward(X, W, b, 6, 1, 0)
    Xf, Wf = X.reshape(7, -1).astype(np.float64), W.reshape(25, -1).astype(np.float64)
    assert maxnorm_rel(Y.reshape(7, 25), (Xf @ Wf.T + b).astype(np.float32)) <= 1e-5
    dX, dW, db = port.conv_backward(X, W, dY, 6, 1, 0)
    g = dY.reshape(7, 25).astype(np.float64)
    assert maxnorm_rel(dX.reshape(7, -1), (g @ Wf).astype(np.float32)) <= 1e-5
    assert maxnorm_rel(dW.reshape(25, -1), (g.T @ Xf).astype(np.float32)) <= 1e-5
    assert maxnorm_rel(db, g.sum(0).astype(np.float32)) <= 1e-5


def test_fp32_and_fp64_accumulation_agree(port):
    X, W, b, dY = make_inputs(6, 2, 8, 9, 12, 5, 1, 2, 2)
    Y32 = port.conv_forward(X, W, b, 5, 1, 2, 2)
    Y64 = port.conv_forward(X, W, b, 5, 1, 2, 2, acc64=True)
    assert maxnorm_rel(Y32, Y64) <= 1e-5


def test_learning_rate_policies(port):
    assert port.learning_rate("fixed", 0.01, 0.1, 5.0, 2.0) == np.float32(0.01)
    assert abs(port.learning_rate("step", 0.01, 0.1, 5.0, 2.0) - 0.01 * 0.1 ** 2) < 1e-9
    assert abs(port.learning_rate("inv", 0.01, 0.1, 5.0, 2.0, power=0.75) - 0.01 * (1.5) ** -0.75) < 1e-9
