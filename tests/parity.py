"""Shared helpers for parity tests: seeded inputs and the error measures used as gates.

Gate (fp32 path, north-star tolerance 1e-4): max-norm relative error  max|a - r| / max|r|  <= 1e-4 per tensor.
Element-wise relative error is ill-posed where outputs cancel to ~0, so it is reported with an absolute floor:
|a - r| <= 1e-4*|r| + 1e-4*rms(r).
"""
import numpy as np

TOL = 1e-4


def maxnorm_rel(a, r):
    denom = float(np.max(np.abs(r)))
    if denom == 0.0:
        return float(np.max(np.abs(a)))
    return float(np.max(np.abs(a.astype(np.float64) - r.astype(np.float64))) / denom)


def elementwise_ok(a, r, tol=TOL):
    r64 = r.astype(np.float64)
    rms = float(np.sqrt(np.mean(r64 * r64)))
    return bool(np.all(np.abs(a.astype(np.float64) - r64) <= tol * np.abs(r64) + tol * rms))


def assert_close(a, r, name, tol=TOL):
    assert a.shape == r.shape, (name, a.shape, r.shape)
    err = maxnorm_rel(a, r)
    assert err <= tol, "%s: max-norm relative error %.3e > %.1e" % (name, err, tol)
    assert elementwise_ok(a, r, tol), "%s: element-wise check with rms floor failed" % name


def make_inputs(seed, B, D, n, o, k, s, p, g=1, x_dist="normal", bias=True, relu_input=False):
    """Seeded synthetic tensors with the value distributions of the benchmark configs:
    X ~ N(0,1) or U(0,1), W ~ N(0, 0.01), bias ~ N(0, 0.01), dY ~ N(0,1)."""
    m = (n + 2 * p - k) // s + 1
    rng = np.random.default_rng(seed)
    if x_dist == "uniform":
        X = rng.random((B, D, n, n), dtype=np.float32)
    else:
        X = rng.standard_normal((B, D, n, n), dtype=np.float32)
    if relu_input:
        X = np.maximum(X, 0)
    W = (0.01 * rng.standard_normal((o, D // g, k, k))).astype(np.float32)
    b = (0.01 * rng.standard_normal((o,))).astype(np.float32) if bias else None
    dY = rng.standard_normal((B, o, m, m), dtype=np.float32)
    return X, W, b, dY
