"""A prototxt-driven network on the GPU against the reference's CPU bridges chained layer by layer: a CaffeNet-shaped
net at reduced width (every layer type and every fusion pattern of CaffeNet: conv+ReLU+pool with LRN behind it,
conv+ReLU feeding a convolution, grouped convolutions, fc+ReLU+dropout feeding an fc, softmax loss), one full training
iteration.  Checked: every layer's output, every parameter gradient, the loss, the updated parameters; the fused net
against the unfused one (same kernels, separate bridges); the model file round trip.  Dropout masks are the ones the
reference's DropoutBridge drew."""
import os

import numpy as np
import pytest

from caffecontroll_b200.net import Net, parse_prototxt, solver_from_message
from oracle import pyoracle
from tests.parity import assert_close, maxnorm_rel

pytestmark = pytest.mark.gpu

NET = """
name: "MiniCaffeNet"
layer { name: "data" type: "Data" top: "data" top: "label" transform_param { crop_size: 67 } }
layer { name: "conv1" type: "Convolution" bottom: "data" top: "conv1" param { lr_mult: 1 decay_mult: 1 } param { lr_mult: 2 decay_mult: 0 }
  convolution_param { num_output: 16 kernel_size: 11 stride: 4 weight_filler { type: "gaussian" std: 0.05 } bias_filler { type: "constant" value: 0 } } }
layer { name: "relu1" type: "ReLU" bottom: "conv1" top: "conv1" }
layer { name: "pool1" type: "Pooling" bottom: "conv1" top: "pool1" pooling_param { pool: MAX kernel_size: 3 stride: 2 } }
layer { name: "norm1" type: "LRN" bottom: "pool1" top: "norm1" lrn_param { local_size: 5 alpha: 0.01 beta: 0.75 } }
layer { name: "conv2" type: "Convolution" bottom: "norm1" top: "conv2" param { lr_mult: 1 decay_mult: 1 } param { lr_mult: 2 decay_mult: 0 }
  convolution_param { num_output: 32 pad: 2 kernel_size: 5 group: 2 weight_filler { type: "gaussian" std: 0.05 } bias_filler { type: "constant" value: 0.1 } } }
layer { name: "relu2" type: "ReLU" bottom: "conv2" top: "conv2" }
layer { name: "conv3" type: "Convolution" bottom: "conv2" top: "conv3" param { lr_mult: 1 decay_mult: 1 } param { lr_mult: 2 decay_mult: 0 }
  convolution_param { num_output: 24 pad: 1 kernel_size: 3 weight_filler { type: "gaussian" std: 0.05 } bias_filler { type: "constant" value: 0 } } }
layer { name: "relu3" type: "ReLU" bottom: "conv3" top: "conv3" }
layer { name: "pool3" type: "Pooling" bottom: "conv3" top: "pool3" pooling_param { pool: MAX kernel_size: 3 stride: 2 } }
layer { name: "fc6" type: "InnerProduct" bottom: "pool3" top: "fc6" param { lr_mult: 1 decay_mult: 1 } param { lr_mult: 2 decay_mult: 0 }
  inner_product_param { num_output: 64 weight_filler { type: "gaussian" std: 0.05 } bias_filler { type: "constant" value: 0.1 } } }
layer { name: "relu6" type: "ReLU" bottom: "fc6" top: "fc6" }
layer { name: "drop6" type: "Dropout" bottom: "fc6" top: "fc6" dropout_param { dropout_ratio: 0.5 } }
layer { name: "fc7" type: "InnerProduct" bottom: "fc6" top: "fc7" param { lr_mult: 1 decay_mult: 1 } param { lr_mult: 2 decay_mult: 0 }
  inner_product_param { num_output: 48 weight_filler { type: "gaussian" std: 0.05 } bias_filler { type: "constant" value: 0.1 } } }
layer { name: "relu7" type: "ReLU" bottom: "fc7" top: "fc7" }
layer { name: "fc8" type: "InnerProduct" bottom: "fc7" top: "fc8" param { lr_mult: 1 decay_mult: 1 } param { lr_mult: 2 decay_mult: 0 }
  inner_product_param { num_output: 12 weight_filler { type: "gaussian" std: 0.05 } bias_filler { type: "constant" value: 0 } } }
layer { name: "loss" type: "SoftmaxWithLoss" bottom: "fc8" bottom: "label" top: "loss" }
"""
SOLVER = 'base_lr: 0.01 lr_policy: "step" gamma: 0.1 stepsize: 1000 momentum: 0.9 weight_decay: 0.0005 random_seed: 3'
B = 8


def _reference_iteration(ref, port, params, X, labels, mask6):
    """The same iteration through the reference's CPU bridges, one bridge at a time (grouped layers per channel slice,
    as the oracle does everywhere).  Returns blobs, gradients and the loss."""
    out, grads = {}, {}
    conv = lambda x, name, k, s, p, g: ref.conv_fwd_bwd(x, params[name][0], params[name][1], np.zeros(
        (x.shape[0], params[name][0].shape[0], (x.shape[2] + 2 * p - k) // s + 1, (x.shape[2] + 2 * p - k) // s + 1), np.float32),
        k, s, p, g=g, needs_dx=False)[0]
    out["conv1"] = ref.relu(conv(X, "conv1", 11, 4, 0, 1))[0]
    out["pool1"], idx1, _ = ref.maxpool(out["conv1"], 3, 2)
    out["norm1"] = ref.lrn(out["pool1"], 5, 0.01, 0.75)[0]
    out["conv2"] = ref.relu(conv(out["norm1"], "conv2", 5, 1, 2, 2))[0]
    out["conv3"] = ref.relu(conv(out["conv2"], "conv3", 3, 1, 1, 1))[0]
    out["pool3"], idx3, _ = ref.maxpool(out["conv3"], 3, 2)
    fc6 = ref.fc(out["pool3"], params["fc6"][0], params["fc6"][1])[0]
    out["fc6"] = (np.maximum(fc6, 0) * mask6 * np.float32(2.0)).astype(np.float32)
    out["fc7"] = np.maximum(ref.fc(out["fc6"], params["fc7"][0].reshape(48, 64, 1, 1), params["fc7"][1])[0], 0)
    out["fc8"] = ref.fc(out["fc7"], params["fc8"][0].reshape(12, 48, 1, 1), params["fc8"][1])[0]
    prob, loss, d8, _ = ref.softmax_loss(out["fc8"], labels)
    # backward
    _, d7, dW, db, _ = ref.fc(out["fc7"], params["fc8"][0].reshape(12, 48, 1, 1), params["fc8"][1], dY=d8)
    grads["fc8"] = (dW, db)
    d7 = d7 * (out["fc7"] > 0)
    _, d6, dW, db, _ = ref.fc(out["fc6"], params["fc7"][0].reshape(48, 64, 1, 1), params["fc7"][1], dY=d7)
    grads["fc7"] = (dW, db)
    d6 = (d6 * mask6 * np.float32(2.0) * (out["fc6"] > 0)).astype(np.float32)
    _, dp3, dW, db, _ = ref.fc(out["pool3"], params["fc6"][0], params["fc6"][1], dY=d6)
    grads["fc6"] = (dW, db)
    d3 = ref.relu(out["conv3"], dY=ref.maxpool(out["conv3"], 3, 2, dY=dp3)[2])[1]
    _, d2, dW, db = ref.conv_fwd_bwd(out["conv2"], params["conv3"][0], params["conv3"][1], d3, 3, 1, 1)
    grads["conv3"] = (dW, db)
    d2 = ref.relu(out["conv2"], dY=d2)[1]
    _, dn1, dW, db = ref.conv_fwd_bwd(out["norm1"], params["conv2"][0], params["conv2"][1], d2, 5, 1, 2, g=2)
    grads["conv2"] = (dW, db)
    dp1 = ref.lrn(out["pool1"], 5, 0.01, 0.75, dY=dn1)[1]
    d1 = ref.relu(out["conv1"], dY=ref.maxpool(out["conv1"], 3, 2, dY=dp1)[2])[1]
    _, _, dW, db = ref.conv_fwd_bwd(X, params["conv1"][0], params["conv1"][1], d1, 11, 4, 0, needs_dx=False)
    grads["conv1"] = (dW, db)
    return out, grads, loss


@pytest.fixture(scope="module")
def nets(ctx):
    net_param, solver = parse_prototxt(NET), solver_from_message(parse_prototxt(SOLVER))
    fused = Net(ctx, net_param, solver, B, fuse=True)
    plain = Net(ctx, net_param, solver, B, fuse=False)
    yield fused, plain
    fused.close()
    plain.close()


def test_net_structure_and_fusions(nets):
    fused, plain = nets
    assert [n for n, _ in fused.param_bridges()] == ["conv1", "conv2", "conv3", "fc6", "fc7", "fc8"]
    assert plain.fused == []
    text = " | ".join(fused.fused)
    assert "conv1+relu1(+pool1 backward)" in text and "conv2+relu2, mask in conv3" in text
    assert "conv3+relu3(+pool3 backward)" in text and "fc6+relu6+drop6, masks in fc7" in text and "fc7+relu7, mask in fc8" in text
    assert fused.num_parameters() == plain.num_parameters() == sum(
        int(np.prod(s)) for s in ((16, 3, 11, 11), (16,), (32, 8, 5, 5), (32,), (24, 32, 3, 3), (24,), (64, 24 * 9), (64,),
                                  (48, 64), (48,), (12, 48), (12,)))
    # same seed -> both nets were filled with the same weights, as every bridge of the reference is
    for (_, a), (_, b) in zip(fused.param_bridges(), plain.param_bridges()):
        assert np.array_equal(a.get_model_cube().download(), b.get_model_cube().download())


def test_iteration_matches_reference_bridges_and_unfused_net(ctx, nets, reference, port, tmp_path):
    fused, plain = nets
    rng = np.random.default_rng(123)
    X = rng.standard_normal((B, 3, 67, 67), dtype=np.float32)
    labels = rng.integers(0, 12, B).astype(np.float32)
    # the reference's DropoutBridge draws the mask; both GPU nets get that one
    _, mask6, _, _ = reference.dropout(np.zeros((B, 64, 1, 1), np.float32), 0.5, 3)
    path = os.path.join(str(tmp_path), "model.bin")
    fused.write_model_to_file(path)
    plain.read_model_from_file(path)
    assert os.path.getsize(path) == 4 * fused.num_parameters()
    params = {n: (pb.get_model_cube().download(), pb.get_bias_cube().download().reshape(-1)) for n, pb in fused.param_bridges()}
    ref_out, ref_grads, ref_loss = _reference_iteration(reference, port, params, X, labels, mask6)
    for net in (fused, plain):
        for i, br in enumerate(net.bridges):
            if net.types[i] == "Dropout":
                br.set_mask(mask6)
        net.set_input(X, labels)
        net.set_update_model_gradients(False)
        net.step()
        ctx.sync()
    for name in ("conv1", "pool1", "norm1", "conv2", "conv3", "pool3", "fc6", "fc7", "fc8"):
        for net, tag in ((fused, "fused"), (plain, "unfused")):
            assert_close(net.blob(name), ref_out[name], "%s %s" % (tag, name))
    for net in (fused, plain):
        assert abs(net.get_loss() - ref_loss) <= 1e-4 * abs(ref_loss)
    for (name, pf), (_, pp) in zip(fused.param_bridges(), plain.param_bridges()):
        dWr, dbr = ref_grads[name]
        for net_pb, tag in ((pf, "fused"), (pp, "unfused")):
            assert_close(net_pb.get_model_grad_cube().download().reshape(dWr.shape), dWr, "%s dW %s" % (tag, name))
            assert_close(net_pb.get_bias_grad_cube().download().reshape(-1), dbr, "%s db %s" % (tag, name))
    # the SGD step: w -= lr * (g + lambda w) on the first iteration (history starts at zero); lr_mult 1 / 2, decay 1 / 0
    for net in (fused, plain):
        net.set_update_model_gradients(True)
        net.step()
        ctx.sync()
    for name, pb in fused.param_bridges():
        W0, b0 = params[name]
        dWr, dbr = ref_grads[name]
        want_W = W0 - np.float32(0.01) * (dWr.reshape(W0.shape) + np.float32(0.0005) * W0)
        want_b = b0 - np.float32(0.02) * dbr
        assert_close(pb.get_model_cube().download().reshape(W0.shape), want_W.astype(np.float32), "updated W " + name)
        assert_close(pb.get_bias_cube().download().reshape(-1), want_b.astype(np.float32), "updated bias " + name)
    for (name, pf), (_, pp) in zip(fused.param_bridges(), plain.param_bridges()):
        assert maxnorm_rel(pf.get_model_cube().download(), pp.get_model_cube().download()) <= 1e-5


def test_snapshot_round_trip_resumes_the_same_trajectory(ctx, tmp_path):
    """MODEL / HISTORY / ITER written after two steps and read into a fresh net: the third step is bit-identical."""
    net_param, solver = parse_prototxt(NET), solver_from_message(parse_prototxt(SOLVER))
    rng = np.random.default_rng(77)
    X = rng.standard_normal((B, 3, 67, 67), dtype=np.float32)
    labels = rng.integers(0, 12, B).astype(np.float32)
    mask = (rng.random((B, 64, 1, 1)) < 0.5).astype(np.uint32)
    a, b = Net(ctx, net_param, solver, B), Net(ctx, net_param, solver, B)
    for net in (a, b):
        for i, br in enumerate(net.bridges):
            if net.types[i] == "Dropout":
                br.set_mask(mask)
        net.set_input(X, labels)
    a.step()
    a.step()
    prefix = os.path.join(str(tmp_path), "snap")
    a.write_snapshot(prefix)
    assert open(prefix + ".ITER").read().split() == ["2"]
    assert os.path.getsize(prefix + ".HISTORY") == os.path.getsize(prefix + ".MODEL") == 4 * a.num_parameters()
    b.read_snapshot(prefix)
    a.step()
    b.step()
    ctx.sync()
    for (name, pa), (_, pb) in zip(a.param_bridges(), b.param_bridges()):
        assert np.array_equal(pa.get_model_cube().download(), pb.get_model_cube().download()), name
        assert np.array_equal(pa.history_host()[0], pb.history_host()[0]), name
    a.close()
    b.close()


def test_l1_solver_and_asynchronous_loss_read(ctx, port):
    """regularization_type "L1" from the solver text reaches the update (g += lambda * sign(w), DeviceDriver::L1_update),
    and read_loss_into() delivers the same number as get_loss() without a stream synchronisation of its own."""
    import ctypes as C
    from caffecontroll_b200 import capi
    net_param = parse_prototxt(NET)
    rng = np.random.default_rng(78)
    X = rng.standard_normal((B, 3, 67, 67), dtype=np.float32)
    labels = rng.integers(0, 12, B).astype(np.float32)
    mask = (rng.random((B, 64, 1, 1)) < 0.5).astype(np.uint32)
    nets = []
    for reg in ("L2", "L1"):
        net = Net(ctx, net_param, solver_from_message(parse_prototxt(SOLVER + ' regularization_type: "%s"' % reg)), B)
        for i, br in enumerate(net.bridges):
            if net.types[i] == "Dropout":
                br.set_mask(mask)
        net.set_input(X, labels)
        nets.append(net)
    l2, l1 = nets
    w0 = {n: pb.get_model_cube().download().copy() for n, pb in l1.param_bridges()}
    host = C.c_void_p()
    capi.check(ctx.lib.cct_malloc_host(ctx.h, 4, C.byref(host)), "cct_malloc_host", ctx.h)
    for net in nets:
        net.step()
    l1.read_loss_into(host.value)
    ctx.sync()
    assert C.c_float.from_address(host.value).value == np.float32(l1.get_loss())
    capi.check(ctx.lib.cct_free_host(ctx.h, host), "cct_free_host", ctx.h)
    # same gradients in both nets (same weights, inputs, masks); the weight updates differ by the regulariser alone:
    # first step, zero history: w1 = w0 - lr * (g + lambda * r(w0)), r = w0 (L2) or sign(w0) with sign(0) = -1 (L1)
    lr, lam = np.float32(0.01), np.float32(0.0005)
    for (name, p1), (_, p2) in zip(l1.param_bridges(), l2.param_bridges()):
        w = w0[name]
        sign = np.where(w > 0, np.float32(1), np.float32(-1))
        want = p2.get_model_cube().download() + lr * lam * (w - sign)
        assert maxnorm_rel(p1.get_model_cube().download(), want) < 1e-6, name
    for net in nets:
        net.close()
