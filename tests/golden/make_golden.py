"""Generates tests/golden/conv_golden.npz from the REFERENCE's own compiled CPU code (oracle/_ref, built by
oracle/build.py from the reference source tree).  Run where the reference tree is mounted:

    python tests/golden/make_golden.py

Each case stores the seeded inputs and what the reference's ParallelizedBridge<ConvolutionBridge> /
MaxPoolingBridge / ReLUBridge produced for them, so that machines without the reference tree can still check
against the reference's results.  Cases are small on purpose (the whole file stays below ~300 KB).
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import build, pyoracle  # noqa: E402
from tests.parity import make_inputs  # noqa: E402

# name: (B, D, n, o, k, s, p, g, partitions, x_dist)
CASES = {
    "ref_small_fixture_shape": (4, 3, 20, 10, 5, 4, 2, 1, 1, "normal"),   # shape of the reference's conv_* fixtures
    "lenet_conv1_small": (2, 1, 16, 20, 5, 1, 0, 1, 2, "uniform"),       # LeNet conv1 filters on a 16x16 crop
    "alexnet_conv1_tiny": (2, 3, 35, 8, 11, 4, 0, 1, 2, "normal"),        # 11x11 stride 4
    "caffenet_conv2_tiny": (2, 8, 9, 12, 5, 1, 2, 2, 1, "normal"),        # 5x5 pad 2, 2 groups
    "conv3_tiny": (3, 6, 7, 10, 3, 1, 1, 1, 1, "normal"),                 # 3x3 pad 1
    "stride2_pad1": (2, 4, 11, 6, 3, 2, 1, 1, 1, "normal"),
    "full_kernel_is_fc": (3, 4, 6, 9, 6, 1, 0, 1, 1, "normal"),           # k = n: convolution == fully connected
}


def main():
    build.build_reference()
    ref = pyoracle.reference()
    if ref is None:
        raise SystemExit("reference library not available")
    out = {}
    for i, (name, (B, D, n, o, k, s, p, g, parts, dist)) in enumerate(CASES.items()):
        X, W, b, dY = make_inputs(100 + i, B, D, n, o, k, s, p, g, x_dist=dist)
        Y, dX, dW, db = ref.conv_fwd_bwd(X, W, b, dY, k, s, p, g=g, partitions=parts)
        out[name + "/shape"] = np.array([B, D, n, o, k, s, p, g], np.int32)
        for key, val in (("X", X), ("W", W), ("b", b), ("dY", dY), ("Y", Y), ("dX", dX), ("dW", dW), ("db", db)):
            out[name + "/" + key] = val
    # SGD step on the fixture shape: lr 0.01, momentum 0.9 (two steps so the history matters), decay 0.0005
    B, D, n, o, k, s, p, g, parts, dist = CASES["ref_small_fixture_shape"]
    X, W, b, dY = make_inputs(100, B, D, n, o, k, s, p, g)
    h = ref.conv_create(B, D, n, o, k, s, p, True, 1, True, 0.01, 0.9, 0.0005)
    ref.lib.cctref_conv_set_model(h, pyoracle._p(W), pyoracle._p(b))
    Yt = np.empty((B, o, 5, 5), np.float32)
    for _ in range(2):
        ref.lib.cctref_conv_forward(h, pyoracle._p(X), pyoracle._p(Yt))
        ref.lib.cctref_conv_backward(h, pyoracle._p(dY), None, None, None, 1)
    W2, b2 = np.empty_like(W), np.empty_like(b)
    ref.lib.cctref_conv_get_model(h, pyoracle._p(W2), pyoracle._p(b2))
    ref.conv_destroy(h)
    out["sgd_two_steps/W"] = W2
    out["sgd_two_steps/b"] = b2
    # pooling + ReLU masks (CaffeNet's 3x3 stride 2, and the reference test's 4x4 stride 2)
    rng = np.random.default_rng(7)
    for name, (B, D, n, k, s) in {"pool3s2": (2, 3, 13, 3, 2), "pool4s2": (2, 3, 10, 4, 2)}.items():
        A = rng.standard_normal((B, D, n, n), dtype=np.float32)
        m = (n - k) // s + 1
        dP = rng.standard_normal((B, D, m, m), dtype=np.float32)
        Yp, idx, dA = ref.maxpool(A, k, s, dP)
        R, dR = ref.relu(A, dA)
        out[name + "/shape"] = np.array([B, D, n, k, s], np.int32)
        for key, val in (("A", A), ("dP", dP), ("Y", Yp), ("idx", idx), ("dA_pool", dA), ("relu", R), ("dA_pool_relu", dR)):
            out[name + "/" + key] = val
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "conv_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes;", len(out), "arrays")


if __name__ == "__main__":
    main()
