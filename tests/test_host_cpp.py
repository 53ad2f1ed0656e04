"""The C++ mirror of the reference's bridge interface (caffecontroll_b200/host/cct_host.h): it must compile and link
against the C ABI alone (CPU check), and on a GPU produce what the CPU oracle produces for the same files."""
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from tests.parity import TOL, assert_close, make_inputs, maxnorm_rel  # noqa: E402


def _build():
    from caffecontroll_b200 import _build
    _build.build()
    return _build.build_host_selftest()


def test_host_mirror_compiles_and_links_against_the_c_abi_only():
    exe = _build()
    assert os.path.exists(exe)
    with open(os.path.join(ROOT, "caffecontroll_b200", "host", "cct_host.h")) as f:
        text = f.read()
    assert "cuda" not in text.lower().replace("cuda_stream", "")  # no CUDA headers or types: plain C ABI
    out = subprocess.run([exe], capture_output=True, text=True)
    assert out.returncode == 2 and "usage" in out.stderr


@pytest.mark.gpu
def test_host_mirror_matches_oracle(port, tmp_path):
    exe = _build()
    B, D, n, o, k, s, p, g = 4, 6, 13, 10, 3, 1, 1, 2
    X, W, b, dY = make_inputs(55, B, D, n, o, k, s, p, g)
    for name, arr in (("X", X), ("W", W), ("b", b), ("dY", dY)):
        arr.tofile(os.path.join(str(tmp_path), name + ".bin"))
    steps = 2
    subprocess.run([exe, str(tmp_path)] + [str(v) for v in (B, D, n, o, k, s, p, g, steps)], check=True)
    rd = lambda name, shape: np.fromfile(os.path.join(str(tmp_path), name + ".bin"), np.float32).reshape(shape)
    m = (n + 2 * p - k) // s + 1
    Yr = port.conv_forward(X, W, b, k, s, p, g)
    dXr, dWr, dbr = port.conv_backward(X, W, dY, k, s, p, g)
    assert_close(rd("Y", (B, o, m, m)), Yr, "Y")
    assert_close(rd("dX", X.shape), dXr, "dX")
    assert_close(rd("dW", W.shape), dWr, "dW")
    assert_close(rd("db", (o,)), dbr, "db")
    Wc, bc = W.copy(), b.copy()
    hw, hb = np.zeros_like(W), np.zeros_like(b)
    for it in range(1, steps + 1):
        _, dW, db = port.conv_backward(X, Wc, dY, k, s, p, g, needs_dx=False)
        lr = port.learning_rate("step", 0.01, 0.1, float(it), 100000.0)
        port.sgd_update(Wc, dW, hw, lr, 0.9, 0.0005)
        port.sgd_update(bc, db, hb, float(np.float32(lr * 2.0)), 0.9, 0.0)
    assert maxnorm_rel(rd("Wnew", W.shape), Wc) <= TOL
    assert maxnorm_rel(rd("bnew", (o,)), bc) <= TOL


@pytest.mark.gpu
def test_host_fully_connected_mirror_matches_oracle(port, tmp_path):
    """kernel == input, so the layer is an inner product: the C++ FullyConnectedBridge mirror must reproduce what the
    ConvolutionBridge mirror (and the oracle) give for it."""
    exe = _build()
    B, D, n, o, k, s, p, g = 6, 5, 4, 12, 4, 1, 0, 1
    X, W, b, dY = make_inputs(56, B, D, n, o, k, s, p, g)
    for name, arr in (("X", X), ("W", W), ("b", b), ("dY", dY)):
        arr.tofile(os.path.join(str(tmp_path), name + ".bin"))
    subprocess.run([exe, str(tmp_path)] + [str(v) for v in (B, D, n, o, k, s, p, g, 0)] + ["fc"], check=True)
    rd = lambda name, shape: np.fromfile(os.path.join(str(tmp_path), name + ".bin"), np.float32).reshape(shape)
    Yr = port.conv_forward(X, W, b, k, s, p, g)
    dXr, dWr, dbr = port.conv_backward(X, W, dY, k, s, p, g)
    for tag in ("", "_fc"):
        assert_close(rd("Y" + tag, (B, o, 1, 1)), Yr, "Y" + tag)
        assert_close(rd("dX" + tag, X.shape), dXr, "dX" + tag)
        assert_close(rd("dW" + tag, W.shape), dWr, "dW" + tag)
        assert_close(rd("db" + tag, (o,)), dbr, "db" + tag)


@pytest.mark.gpu
def test_host_mirror_two_gpus_one_thread_each(port, tmp_path):
    """The C++ ParallelizedBridge with the C ABI's NCCL communicator, no Python and no torch in the data path: two host
    threads, one GPU each, half the batch each; after two SGD steps both hold the parameters of the single-GPU run."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    exe = _build()
    B, D, n, o, k, s, p, g = 8, 6, 13, 10, 3, 1, 1, 1
    X, W, b, dY = make_inputs(57, B, D, n, o, k, s, p, g)
    for name, arr in (("X", X), ("W", W), ("b", b), ("dY", dY)):
        arr.tofile(os.path.join(str(tmp_path), name + ".bin"))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    subprocess.run([exe, str(tmp_path)] + [str(v) for v in (B, D, n, o, k, s, p, g, 2)] + ["ranks=2"], check=True, env=env,
                   timeout=300)
    rd = lambda name, shape: np.fromfile(os.path.join(str(tmp_path), name + ".bin"), np.float32).reshape(shape)
    W1, b1 = rd("Wnew", W.shape), rd("bnew", (o,))
    for r in (0, 1):
        assert maxnorm_rel(rd("Wnew_r%d" % r, W.shape), W1) <= TOL
        assert maxnorm_rel(rd("bnew_r%d" % r, (o,)), b1) <= TOL
    assert np.array_equal(rd("Wnew_r0", W.shape), rd("Wnew_r1", W.shape))


@pytest.mark.gpu
def test_host_mirror_model_parallel_fc_two_gpus(port, tmp_path):
    """The C++ ModelParallelFullyConnectedBridge (output depth split over two GPUs, one host thread each, NCCL exchanges
    through the C ABI): every rank's output rows, input-gradient rows and its slice of the weight and bias gradients
    against the oracle's product over the whole batch."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    exe = _build()
    B, D, n, o, k, s, p, g = 8, 5, 4, 24, 4, 1, 0, 1
    X, W, b, dY = make_inputs(58, B, D, n, o, k, s, p, g)
    for name, arr in (("X", X), ("W", W), ("b", b), ("dY", dY)):
        arr.tofile(os.path.join(str(tmp_path), name + ".bin"))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    subprocess.run([exe, str(tmp_path)] + [str(v) for v in (B, D, n, o, k, s, p, g, 0)] + ["mpfc=2"], check=True, env=env,
                   timeout=300)
    rd = lambda name, shape: np.fromfile(os.path.join(str(tmp_path), name + ".bin"), np.float32).reshape(shape)
    Yr = port.conv_forward(X, W, b, k, s, p, g)
    dXr, dWr, dbr = port.conv_backward(X, W, dY, k, s, p, g)
    Bp, os_ = B // 2, o // 2
    for r in (0, 1):
        rows, cols = slice(r * Bp, (r + 1) * Bp), slice(r * os_, (r + 1) * os_)
        assert_close(rd("Y_mp%d" % r, (Bp, o, 1, 1)), Yr[rows], "Y rank %d" % r)
        assert_close(rd("dX_mp%d" % r, (Bp,) + X.shape[1:]), dXr[rows], "dX rank %d" % r)
        assert_close(rd("dW_mp%d" % r, (os_,) + W.shape[1:]), dWr[cols], "dW rank %d" % r)
        assert_close(rd("db_mp%d" % r, (os_,)), dbr[cols], "db rank %d" % r)

