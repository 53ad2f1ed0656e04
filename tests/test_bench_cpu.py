"""CPU checks of bench.py's bookkeeping: the layer table of the reference arm against the network description the GPU arm
builds, the FLOP count behind the roofline, and the measured-traffic look-up."""
import json
import os

import bench
from caffecontroll_b200.net import parse_prototxt

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _prototxt_layers():
    with open(os.path.join(ROOT, "caffecontroll_b200", "nets", "caffenet_train.prototxt")) as f:
        net = parse_prototxt(f.read())
    return [l for l in net.all("layer") if l.get1("type") not in ("Data", "Accuracy")]


def test_reference_arm_layer_table_matches_the_prototxt():
    table = bench.caffenet_layer_table()
    layers = _prototxt_layers()
    assert [name for name, _, _ in table] == [l.get1("name") for l in layers]
    kinds = {"Convolution": "conv", "ReLU": "relu", "Pooling": "pool", "LRN": "lrn", "InnerProduct": "fc",
             "Dropout": "dropout", "SoftmaxWithLoss": "softmax"}
    for (name, kind, geo), layer in zip(table, layers):
        assert kinds[layer.get1("type")] == kind, name
        if kind == "conv":
            cp = layer.msg("convolution_param")
            assert (geo["o"], geo["k"], geo["s"], geo["p"], geo["g"]) == (
                cp.get1("num_output"), cp.get1("kernel_size"), cp.get1("stride", 1), cp.get1("pad", 0), cp.get1("group", 1)), name
        if kind == "fc":
            assert geo["o"] == layer.msg("inner_product_param").get1("num_output"), name


def test_flops_per_iteration_at_batch_256():
    # 2 * multiply-adds of every contraction, three contractions per parameterised layer except conv1 (no dX)
    total = 0.0
    for name, kind, g in bench.caffenet_layer_table():
        if kind == "conv":
            m = (g["n"] + 2 * g["p"] - g["k"]) // g["s"] + 1
            f = 2.0 * g["o"] * (g["k"] ** 2 * g["D"] // g["g"]) * m * m * 256
            total += f * (3 if g["needs_dx"] else 2)
        elif kind == "fc":
            total += 3 * 2.0 * g["o"] * g["D"] * g["n"] * g["n"] * 256
    assert abs(total / 1e9 - 1058.7) < 0.1


def test_traffic_lookup_scales_with_batch_and_misses_cleanly():
    with open(os.path.join(ROOT, "profiles", "dram_traffic.json")) as f:
        table = json.load(f)
    e = table["caffenet"]["conv2 data gradient"]
    full, source = bench.caffenet_traffic("conv2 dgrad", 256)
    assert full == e["dram_read_bytes"] + e["dram_write_bytes"] and source.startswith("profiles/")
    assert os.path.exists(os.path.join(ROOT, source))
    half, _ = bench.caffenet_traffic("conv2 dgrad", 128)
    assert abs(half - full / 2) < 1.0
    assert bench.caffenet_traffic("fc6 forward", 256)[0] > 150e6   # the layer's weights cross HBM once
    assert bench.caffenet_traffic("conv9 wgrad", 256) == (None, None)
