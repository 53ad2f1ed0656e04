"""GPU test of cct_conv_weight_grad_noalloc, the entry point for callers that may not allocate device memory when
they call (a pool already owns the device, a latency-critical section, allocator hooks that forbid it).  Such callers
cannot build a plan, so the call keeps its scratch in a fixed array inside the library.  Checked here through the
C ABI against the plan-based cct_conv_backward on the same inputs, twice in a row (the second call reuses the array
with the first call's leftovers in it), against the CPU oracle on layers whose pixel count needs many splits (bounded
accumulation chains) and more splits than the array holds at once (several rounds over the same slices), and for a
layer that exceeds the limit.

The file name sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

from tests.parity import assert_close, make_inputs

pytestmark = pytest.mark.gpu


def _upload(ctx, arr):
    ptr = ctx.malloc(arr.nbytes)
    ctx.h2d(ptr, arr)
    return ptr


def _download(ctx, ptr, shape):
    out = np.empty(shape, np.float32)
    ctx.d2h(out, ptr)
    return out


def _plan_weight_grad(ctx, capi, desc, pX, pW, pdY, w_shape, o):
    """dW, db from the existing entry point (plan + cct_conv_backward without a data gradient)."""
    lib = ctx.lib
    plan = C.c_void_p()
    capi.check(lib.cct_conv_plan_create(ctx.h, C.byref(desc), C.byref(plan)), "cct_conv_plan_create", ctx.h)
    pdW, pdb = ctx.malloc(4 * int(np.prod(w_shape))), ctx.malloc(4 * o)
    capi.check(lib.cct_conv_backward(plan, C.c_void_p(pX), C.c_void_p(pW), C.c_void_p(pdY), None, C.c_void_p(pdW),
                                     C.c_void_p(pdb)), "cct_conv_backward", ctx.h)
    ctx.sync()
    lib.cct_conv_plan_destroy(plan)
    dW, db = _download(ctx, pdW, w_shape), _download(ctx, pdb, (o,))
    ctx.free(pdW)
    ctx.free(pdb)
    return dW, db


@pytest.mark.parametrize("shape", [(6, 16, 14, 24, 3, 1, 1, 1), (4, 3, 35, 8, 11, 4, 0, 1), (3, 8, 9, 12, 5, 1, 2, 2)])
def test_noalloc_weight_gradient_matches_plan_path_twice(ctx, shape):
    from caffecontroll_b200 import capi
    lib = ctx.lib
    B, D, n, o, k, s, p, g = shape
    desc = capi.ConvDesc(B, D, n, o, k, s, p, g, 1, capi.ALGO_UMMA_3XTF32)
    for seed in (31, 32):  # two calls in a row, different data: the array keeps the first call's contents
        X, W, b, dY = make_inputs(seed, B, D, n, o, k, s, p, g)
        pX, pW, pdY = _upload(ctx, X), _upload(ctx, W), _upload(ctx, dY)
        want_dW, want_db = _plan_weight_grad(ctx, capi, desc, pX, pW, pdY, W.shape, o)
        pdW, pdb = ctx.malloc(W.nbytes), ctx.malloc(4 * o)
        capi.check(lib.cct_conv_weight_grad_noalloc(ctx.h, C.byref(desc), C.c_void_p(pX), C.c_void_p(pdY),
                                                    C.c_void_p(pdW), C.c_void_p(pdb)),
                   "cct_conv_weight_grad_noalloc", ctx.h)
        ctx.sync()
        assert_close(_download(ctx, pdW, W.shape), want_dW, "dW (no-alloc vs plan)")
        assert_close(_download(ctx, pdb, (o,)), want_db, "db (no-alloc vs plan)")
        for ptr in (pX, pW, pdY, pdW, pdb):
            ctx.free(ptr)


def _noalloc(ctx, capi, desc, X, dY, w_shape, o):
    lib = ctx.lib
    pX, pdY = _upload(ctx, X), _upload(ctx, dY)
    pdW, pdb = ctx.malloc(4 * int(np.prod(w_shape))), ctx.malloc(4 * o)
    capi.check(lib.cct_conv_weight_grad_noalloc(ctx.h, C.byref(desc), C.c_void_p(pX), C.c_void_p(pdY), C.c_void_p(pdW),
                                                C.c_void_p(pdb)), "cct_conv_weight_grad_noalloc", ctx.h)
    ctx.sync()
    dW, db = _download(ctx, pdW, w_shape), _download(ctx, pdb, (o,))
    for ptr in (pX, pdY, pdW, pdb):
        ctx.free(ptr)
    return dW, db


# B, D, n, o, k, s, p: 3025 k-blocks of 32 pixels in 74 splits (one round); CaffeNet conv2's per-group shape with 29
# splits of 0.66 MB partial sums, four more than the 16 MiB array holds (two rounds); AlexNet conv1 at the full batch
# of 256 (BASELINE config 2: 24 200 k-blocks = 138 splits of at most 176 k-blocks, 113 fit at once: two rounds).
@pytest.mark.parametrize("shape", [(32, 3, 227, 96, 11, 4, 0), (96, 48, 27, 128, 5, 1, 2), (256, 3, 227, 96, 11, 4, 0)],
                         ids=["conv1_b32", "conv2_group_b96_two_rounds", "conv1_b256"])
def test_noalloc_weight_gradient_matches_cpu_oracle(ctx, reference, shape):
    import warnings
    from caffecontroll_b200 import capi
    from tests.parity import maxnorm_rel
    B, D, n, o, k, s, p = shape
    X, W, b, dY = make_inputs(41, B, D, n, o, k, s, p, 1, relu_input=(D == 48))
    _, _, dWr, dbr = reference.conv_fwd_bwd(X, W, b, dY, k, s, p, partitions=reference.default_partitions(B),
                                            needs_dx=False)
    desc = capi.ConvDesc(B, D, n, o, k, s, p, 1, 1, capi.ALGO_UMMA_3XTF32)
    dW, db = _noalloc(ctx, capi, desc, X, dY, W.shape, o)
    warnings.warn("parity no-alloc weight gradient %s: dW %.2e, db %.2e" % (shape, maxnorm_rel(dW, dWr),
                                                                          maxnorm_rel(db, dbr)))
    assert_close(dW, dWr, "dW (no-alloc vs CPU oracle)")
    assert_close(db, dbr, "db (no-alloc vs CPU oracle)")


def test_noalloc_rejects_layers_beyond_its_scratch(ctx):
    from caffecontroll_b200 import capi
    lib = ctx.lib
    # 512 filters over 512 x 5 x 5 taps: one split of partial sums is ~26 MB, more than the 16 MiB array holds.
    desc = capi.ConvDesc(1, 512, 8, 512, 5, 1, 2, 1, 1, capi.ALGO_UMMA_3XTF32)
    dummy = ctx.malloc(1024)
    rc = lib.cct_conv_weight_grad_noalloc(ctx.h, C.byref(desc), C.c_void_p(dummy), C.c_void_p(dummy),
                                          C.c_void_p(dummy), C.c_void_p(dummy))
    assert rc == capi.CCT_ERR_UNSUPPORTED
    assert b"16777216" in lib.cct_last_error_string(ctx.h)
    ctx.free(dummy)
