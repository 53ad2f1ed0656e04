"""CPU tests of the host logic around the network builder: the protobuf text-format reader on the package's own CaffeNet
description (and, where the reference tree is mounted, on every prototxt the reference ships), solver defaults, per-blob
multipliers in both notations."""
import glob
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from caffecontroll_b200.net import _in_phase, _layer_type, _multipliers, parse_prototxt, solver_from_message  # noqa: E402

NETS = os.path.join(ROOT, "caffecontroll_b200", "nets")


def test_caffenet_description_parses_to_the_published_architecture():
    with open(os.path.join(NETS, "caffenet_train.prototxt")) as f:
        net = parse_prototxt(f.read())
    layers = net.all("layer")
    assert [str(l.get1("name")) for l in layers] == [
        "data", "conv1", "relu1", "pool1", "norm1", "conv2", "relu2", "pool2", "norm2", "conv3", "relu3", "conv4", "relu4",
        "conv5", "relu5", "pool5", "fc6", "relu6", "drop6", "fc7", "relu7", "drop7", "fc8", "loss"]
    conv = {str(l.get1("name")): l.msg("convolution_param") for l in layers if _layer_type(l) == "Convolution"}
    assert [(int(c.get1("num_output")), int(c.get1("kernel_size")), int(c.get1("stride", 1)), int(c.get1("pad", 0)),
             int(c.get1("group", 1))) for c in conv.values()] == [(96, 11, 4, 0, 1), (256, 5, 1, 2, 2), (384, 3, 1, 1, 1),
                                                                   (384, 3, 1, 1, 2), (256, 3, 1, 1, 2)]
    assert _multipliers(layers[1]) == ((1.0, 2.0), (1.0, 0.0))
    lrn = layers[4].msg("lrn_param")
    assert (int(lrn.get1("local_size")), float(lrn.get1("alpha")), float(lrn.get1("beta"))) == (5, 1e-4, 0.75)
    # 60 965 224 parameters in the grouped CaffeNet
    total = 0
    D = 3
    for name, c in conv.items():
        o, k, g = int(c.get1("num_output")), int(c.get1("kernel_size")), int(c.get1("group", 1))
        total += o * (D // g) * k * k + o
        D = o
    total += 4096 * 9216 + 4096 + 4096 * 4096 + 4096 + 1000 * 4096 + 1000
    assert total == 60965224


def test_solver_fields_and_defaults():
    with open(os.path.join(NETS, "caffenet_solver.prototxt")) as f:
        s = solver_from_message(parse_prototxt(f.read()))
    assert (s.base_lr, s.lr_policy, s.gamma, s.stepsize, s.momentum, s.weight_decay, s.random_seed) == \
        (0.005, "step", 0.1, 100000, 0.9, 0.0005, 1)
    d = solver_from_message(parse_prototxt("base_lr: 0.1"))
    assert (d.lr_policy, d.momentum, d.weight_decay, d.regularization_type, d.random_seed) == ("fixed", 0.0, 0.0, "L2", -1)


def test_text_format_details():
    m = parse_prototxt('''
      # a comment
      name: "n"  layers { name: 'a' type: CONVOLUTION blobs_lr: 1 blobs_lr: 2 weight_decay: 1 weight_decay: 0
                          include: { phase: TEST } convolution_param { num_output: 4 kernel_size: 3 pad: 1 } }
      layer { name: "b" type: "InnerProduct" param { lr_mult: 3 } param { lr_mult: 4 decay_mult: 0.5 } vals: [1, 2.5, -3e-2] }
    ''')
    a, b = m.all("layers")[0], m.all("layer")[0]
    assert _layer_type(a) == "Convolution" and _layer_type(b) == "InnerProduct"
    assert not _in_phase(a, "TRAIN") and _in_phase(a, "TEST") and _in_phase(b, "TRAIN")
    assert _multipliers(a) == ((1.0, 2.0), (1.0, 0.0)) and _multipliers(b) == ((3.0, 4.0), (1.0, 0.5))
    assert b.all("vals") == [1, 2.5, -0.03]
    for bad in ("layer { name: 1", "}", "a: { b: 2 } }"):
        with pytest.raises(ValueError):
            parse_prototxt(bad)


def test_every_prototxt_of_the_reference_parses():
    from oracle import build as obuild
    ref = obuild.reference_root()
    files = glob.glob(os.path.join(ref, "tests", "**", "*.prototxt"), recursive=True) + \
        glob.glob(os.path.join(ref, "benchmark", "**", "*.prototxt"), recursive=True)
    if not files:
        pytest.skip("the reference tree is not mounted here")
    for f in files:
        with open(f) as fh:
            m = parse_prototxt(fh.read())
        assert m, f
    with open(os.path.join(ref, "tests", "imagenet_train", "train_val", "caffenet_train_val_1000.prototxt")) as fh:
        layers = [l for l in parse_prototxt(fh.read()).all("layer") if _in_phase(l, "TRAIN")]
    assert [_layer_type(l) for l in layers].count("Convolution") == 5
    assert _multipliers(layers[1]) == ((1.0, 2.0), (1.0, 0.0))  # the older blobs_lr / weight_decay notation


def test_model_parallel_placement_fields_follow_the_reference_rules():
    """DeepNet::get_model_parallelism_info (src/DeepNet.h:728-790)."""
    import pytest
    from caffecontroll_b200.parallel import model_parallel_gpus
    assert model_parallel_gpus([0.0, 0.0, 0.0, 0.0], 4096) == []
    assert model_parallel_gpus([0.5, 0.5, 0.0, 0.0], 4096) == [0, 1]
    assert model_parallel_gpus([0.25, 0.25, 0.25, 0.25], 4096) == [0, 1, 2, 3]
    for bad, depth in (([1.0, 0.0, 0.0, 0.0], 4096),      # one GPU: use batch proportions
                       ([0.5, 0.25, 0.25, 0.0], 4096),     # unequal shares
                       ([0.5, 0.0, 0.0, 0.0], 4096),       # does not add up to 1
                       ([0.5, 0.5, 0.0, 0.0], 1001)):      # does not divide the depth
        with pytest.raises(ValueError):
            model_parallel_gpus(bad, depth)

