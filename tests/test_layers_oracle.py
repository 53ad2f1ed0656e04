"""CPU tests of the oracle for the CaffeNet bridges around the convolution path: the numpy restatements in
oracle/pyoracle.py (LRN, softmax loss, the fully connected products, dropout) against the reference's own compiled
CPU bridges (oracle/_ref).  Tolerances: the reference works in fp32, the restatements in float64."""
import numpy as np
import pytest

from oracle import pyoracle
from tests.parity import assert_close


@pytest.mark.parametrize("shape", [(3, 8, 5, 5), (2, 96, 27, 5), (2, 5, 4, 3)])  # B, D, n, local_size
def test_lrn_restatement_matches_reference(reference, shape):
    B, D, n, local = shape
    rng = np.random.default_rng(3)
    X = np.maximum(rng.standard_normal((B, D, n, n), dtype=np.float32) * 8, 0)  # pooled ReLU outputs: non-negative, large
    dY = rng.standard_normal((B, D, n, n), dtype=np.float32)
    alpha, beta = 1e-1, 0.75  # a large alpha so that the normalisation is far from the identity
    Yr, dXr, _ = reference.lrn(X, local, alpha, beta, dY=dY)
    Y, scale = pyoracle.np_lrn_forward(X, local, alpha, beta)
    assert scale.max() > 2.0
    assert_close(Y, Yr, "LRN forward")
    assert_close(pyoracle.np_lrn_backward(X, dY, local, alpha, beta), dXr, "LRN backward")


def test_softmax_loss_restatement_matches_reference(reference):
    rng = np.random.default_rng(4)
    X = (3 * rng.standard_normal((16, 50, 1, 1))).astype(np.float32)
    labels = rng.integers(0, 50, 16).astype(np.float32)
    pr, lr, gr, _ = reference.softmax_loss(X, labels)
    p, l, g = pyoracle.np_softmax_loss(X, labels)
    assert_close(p, pr, "softmax probabilities")
    assert abs(l - lr) <= 1e-4 * abs(lr)
    assert_close(g, gr, "softmax-loss gradient")


def test_fully_connected_products_match_reference(reference):
    rng = np.random.default_rng(5)
    B, D, n, o = 6, 5, 3, 9
    X = rng.standard_normal((B, D, n, n), dtype=np.float32)
    W = (0.1 * rng.standard_normal((o, D, n, n))).astype(np.float32)
    b = rng.standard_normal(o).astype(np.float32)
    dY = rng.standard_normal((B, o, 1, 1), dtype=np.float32)
    Yr, dXr, dWr, dbr, _ = reference.fc(X, W, b, dY=dY)
    X2, W2, dY2 = X.reshape(B, -1).astype(np.float64), W.reshape(o, -1).astype(np.float64), dY.reshape(B, o).astype(np.float64)
    assert_close((X2 @ W2.T + b).astype(np.float32).reshape(B, o, 1, 1), Yr, "Y = X W^T + b")
    assert_close((dY2 @ W2).astype(np.float32).reshape(X.shape), dXr, "dX = dY W")
    assert_close((dY2.T @ X2).astype(np.float32).reshape(W.shape), dWr, "dW = dY^T X")
    assert_close(dY2.sum(axis=0).astype(np.float32), dbr, "db")


def test_dropout_is_mask_times_scale(reference):
    rng = np.random.default_rng(6)
    X = rng.standard_normal((4, 8, 3, 3), dtype=np.float32)
    dY = rng.standard_normal((4, 8, 3, 3), dtype=np.float32)
    Y, mask, dX, _ = reference.dropout(X, 0.5, 7, dY=dY)
    assert set(np.unique(mask)) <= {0, 1} and 0.2 < mask.mean() < 0.8
    assert np.array_equal(Y, X * mask * np.float32(2.0))
    assert np.array_equal(dX, dY * mask * np.float32(2.0))
