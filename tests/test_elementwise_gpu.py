"""GPU tests of the memory-bound companions (pooling / ReLU masks, SGD step, fill): integer and copy work is
compared bit-exactly, fp32 sums that follow the oracle's order too."""
import ctypes as C
import os

import numpy as np
import pytest

from caffecontroll_b200.bridge import LogicalCube

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "conv_golden.npz")


def _cube(ctx, arr):
    return LogicalCube.from_numpy(ctx, arr)


# (2, 2, 9, 3, 1) and (1, 2, 11, 5, 1) have three and five windows per axis over an element: the kernels for overlapping
# pooling beyond 2x2; the last two are 3x3 stride-2 cases with several plane groups and a ragged last one, and an even size
@pytest.mark.parametrize("shape", [(2, 3, 13, 3, 2), (2, 3, 10, 4, 2), (1, 2, 27, 3, 2), (3, 1, 7, 2, 1), (1, 1, 9, 3, 3),
                                   (2, 2, 9, 3, 1), (1, 2, 11, 5, 1), (5, 7, 55, 3, 2), (2, 5, 12, 3, 2)])
def test_pool_and_relu_masks_match_oracle_bitwise(ctx, port, shape):
    from caffecontroll_b200 import capi
    B, D, n, k, s = shape
    m = (n - k) // s + 1
    rng = np.random.default_rng(21)
    A = rng.standard_normal((B, D, n, n), dtype=np.float32)
    A[0, 0, :3, :3] = 1.5  # ties: the first maximum must win
    dP = rng.standard_normal((B, D, m, m), dtype=np.float32)
    Yr, idxr = port.maxpool_forward(A, k, s)
    dAr = port.maxpool_backward(dP, idxr, n)
    lib = ctx.lib
    cA, cdP = _cube(ctx, A), _cube(ctx, dP)
    cY, cidx = LogicalCube(ctx, m, m, D, B), LogicalCube(ctx, m, m, D, B, np.int32)
    cdA, cdA2, cR, cdR = (LogicalCube(ctx, n, n, D, B) for _ in range(4))
    vp = C.c_void_p
    capi.check(lib.cct_maxpool_forward(ctx.h, vp(cA.ptr), vp(cY.ptr), vp(cidx.ptr), B * D, n, k, s), "pool fwd", ctx.h)
    capi.check(lib.cct_maxpool_backward(ctx.h, vp(cdP.ptr), vp(cidx.ptr), vp(cdA.ptr), B * D, n, k, s), "pool bwd", ctx.h)
    capi.check(lib.cct_pool_relu_backward(ctx.h, vp(cA.ptr), vp(cidx.ptr), vp(cdP.ptr), vp(cdA2.ptr), B * D, n, k, s),
               "pool+relu bwd", ctx.h)
    capi.check(lib.cct_relu_forward(ctx.h, vp(cA.ptr), vp(cR.ptr), A.size), "relu fwd", ctx.h)
    capi.check(lib.cct_relu_backward(ctx.h, vp(cA.ptr), vp(cdA.ptr), vp(cdR.ptr), A.size), "relu bwd", ctx.h)
    ctx.sync()
    assert np.array_equal(cY.download(), Yr)
    assert np.array_equal(cidx.download(), idxr)
    assert np.array_equal(cdA.download(), dAr)
    assert np.array_equal(cR.download(), port.relu_forward(A))
    assert np.array_equal(cdR.download(), port.relu_backward(A, dAr))
    assert np.array_equal(cdA2.download(), port.relu_backward(A, dAr))
    for c in (cA, cdP, cY, cidx, cdA, cdA2, cR, cdR):
        c.free()


def test_pool_backward_takes_pointers_that_are_not_16_byte_aligned(ctx, port):
    """The 3x3 stride-2 kernel reads the pooled tensors in 16-byte pieces only where the caller's pointers allow it."""
    from caffecontroll_b200 import capi
    B, D, n, k, s = 3, 5, 27, 3, 2
    m = (n - k) // s + 1
    rng = np.random.default_rng(5)
    A = rng.standard_normal((B, D, n, n), dtype=np.float32)
    dP = rng.standard_normal((B, D, m, m), dtype=np.float32)
    _, idxr = port.maxpool_forward(A, k, s)
    dAr = port.maxpool_backward(dP, idxr, n)
    pad = lambda a: np.concatenate([np.zeros(1, a.dtype), a.ravel()]).reshape(1, 1, 1, -1)
    cA, cdP, cidx = _cube(ctx, A), _cube(ctx, pad(dP)), _cube(ctx, pad(idxr.astype(np.int32)))
    cdA = LogicalCube(ctx, n, n, D, B)
    lib, vp = ctx.lib, C.c_void_p
    capi.check(lib.cct_maxpool_backward(ctx.h, vp(cdP.ptr + 4), vp(cidx.ptr + 4), vp(cdA.ptr), B * D, n, k, s), "pool bwd", ctx.h)
    ctx.sync()
    assert np.array_equal(cdA.download(), dAr)
    capi.check(lib.cct_pool_relu_backward(ctx.h, vp(cA.ptr), vp(cidx.ptr + 4), vp(cdP.ptr + 4), vp(cdA.ptr), B * D, n, k, s),
               "pool+relu bwd", ctx.h)
    ctx.sync()
    assert np.array_equal(cdA.download(), port.relu_backward(A, dAr))
    for c in (cA, cdP, cidx, cdA):
        c.free()


def test_masks_match_committed_reference_fixtures(ctx):
    from caffecontroll_b200 import capi
    z = np.load(GOLDEN)
    lib, vp = ctx.lib, C.c_void_p
    for name in ("pool3s2", "pool4s2"):
        B, D, n, k, s = (int(v) for v in z[name + "/shape"])
        m = (n - k) // s + 1
        cA, cdP = _cube(ctx, z[name + "/A"]), _cube(ctx, z[name + "/dP"])
        cY, cidx, cdA = LogicalCube(ctx, m, m, D, B), LogicalCube(ctx, m, m, D, B, np.int32), LogicalCube(ctx, n, n, D, B)
        capi.check(lib.cct_maxpool_forward(ctx.h, vp(cA.ptr), vp(cY.ptr), vp(cidx.ptr), B * D, n, k, s), "pool fwd", ctx.h)
        capi.check(lib.cct_pool_relu_backward(ctx.h, vp(cA.ptr), vp(cidx.ptr), vp(cdP.ptr), vp(cdA.ptr), B * D, n, k, s),
                   "pool+relu bwd", ctx.h)
        ctx.sync()
        assert np.array_equal(cY.download(), z[name + "/Y"])
        assert np.array_equal(cidx.download(), z[name + "/idx"])
        assert np.array_equal(cdA.download(), z[name + "/dA_pool_relu"])
        for c in (cA, cdP, cY, cidx, cdA):
            c.free()


def test_sgd_step_matches_oracle_bitwise(ctx, port):
    from caffecontroll_b200 import capi
    rng = np.random.default_rng(22)
    n = 100003
    w, g, h = (rng.standard_normal(n).astype(np.float32) for _ in range(3))
    cw, cg, ch = _cube(ctx, w), _cube(ctx, g), _cube(ctx, h)
    for lam in (0.0005, 0.0):
        capi.check(ctx.lib.cct_sgd_step(ctx.h, n, C.c_void_p(cw.ptr), C.c_void_p(cg.ptr), C.c_void_p(ch.ptr), 0.01, 0.9,
                                        lam), "sgd", ctx.h)
        port.sgd_update(w, g, h, 0.01, 0.9, lam)
    ctx.sync()
    assert np.array_equal(cw.download().ravel(), w)
    assert np.array_equal(cg.download().ravel(), g)
    assert np.array_equal(ch.download().ravel(), h)


def test_l1_regularised_update_matches_reference_rule(ctx, port):
    """regularization_type "L1": g += lambda * (w > 0 ? 1 : -1) (src/sched/DeviceDriver_CPU.cpp:111-117), then the
    momentum step without decay; through DeviceOps.sgd_step, the call ParallelizedBridge makes."""
    from caffecontroll_b200.parallel import DeviceOps
    rng = np.random.default_rng(23)
    n = 70001
    w, g, h = (rng.standard_normal(n).astype(np.float32) for _ in range(3))
    w[::7] = 0.0
    cw, cg, ch = _cube(ctx, w), _cube(ctx, g), _cube(ctx, h)
    lam = np.float32(0.0005)
    DeviceOps(ctx).sgd_step(n, cw.ptr, cg.ptr, ch.ptr, 0.01, 0.9, float(lam), "L1")
    g = (g + np.where(w > 0, lam, -lam)).astype(np.float32)
    port.sgd_update(w, g, h, 0.01, 0.9, 0.0)
    ctx.sync()
    assert np.array_equal(cg.download().ravel(), g)
    assert np.array_equal(ch.download().ravel(), h)
    assert np.array_equal(cw.download().ravel(), w)


def test_fill_and_empty_sizes(ctx):
    from caffecontroll_b200 import capi
    c = LogicalCube(ctx, 5, 7, 3, 2)
    c.reset_cube(-2.5)
    assert np.all(c.download() == np.float32(-2.5))
    assert ctx.lib.cct_fill_f32(ctx.h, None, 0, 1.0) == capi.CCT_OK
    assert ctx.lib.cct_memset(ctx.h, None, 0, 0) == capi.CCT_OK
    c.free()


@pytest.mark.parametrize("kind,a,b,n_batch", [(0, 0.0, 0.01, 1), (0, 0.5, 2.0, 1), (1, 363.0, 0.0, 96), (2, 0.3, 0.0, 1)])
def test_fillers_reproduce_the_reference_fillers(ctx, reference, kind, a, b, n_batch):
    """cct_fill_random against CPUDriver::sgaussian_initialize / sinitialize_xavier / sbernoulli_initialize
    (src/sched/DeviceDriver_CPU.cpp:661-699) with the same seed: the same generator and distributions, so the same
    sequence - bit for bit for the Bernoulli draws, to the last unit or two for the floating-point ones (the checker is
    built with -march=native, whose fused multiply-adds round the distributions' affine maps once instead of twice).
    Xavier: a = fan-in = elements per filter."""
    from caffecontroll_b200 import capi
    count = 96 * 363 if kind == 1 else 50021
    seed = 17
    cube = LogicalCube(ctx, 1, 1, count, 1)
    capi.check(ctx.lib.cct_fill_random(ctx.h, C.c_void_p(cube.ptr), count, kind, a, b, seed), "cct_fill_random", ctx.h)
    got = cube.download().ravel()
    want = reference.fill(kind, count, a=a, b=b, seed=seed, n_batch=n_batch)
    if kind == 2:
        assert np.array_equal(got, want)
    else:
        scale = np.abs(want).max()
        assert np.abs(got - want).max() <= 4e-6 * scale
        assert np.mean(got == want) > 0.5   # the same draws: most values agree exactly, the rest differ in the last place
    cube.free()
