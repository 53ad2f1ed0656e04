"""CPU tests of the ParallelizedBridge mirror (caffecontroll_b200/parallel.py): batch slicing, learning-rate policy,
per-blob multipliers, and the all-reduce + SGD step with two gloo ranks.  The sub-bridge and the device arithmetic are
replaced by the CPU oracle here (test infrastructure); on a GPU the same class drives the CUDA bridge and NCCL."""
import ctypes as C
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from caffecontroll_b200.parallel import (ParallelizedBridge, SolverParameter, get_learning_rate, partition_batch,  # noqa: E402
                                         partition_by_proportions)
from tests.parity import make_inputs, maxnorm_rel  # noqa: E402

SHAPE = (6, 3, 9, 5, 3, 2, 1, 1)  # B, D, n, o, k, s, p, g
LR, MOM, WD = 0.01, 0.9, 0.0005


def test_partition_batch_is_contiguous_and_complete():
    assert partition_batch(2048, 8) == [(256 * i, 256) for i in range(8)]
    assert partition_batch(10, 4) == [(0, 4), (4, 2), (6, 2), (8, 2)]  # leftovers go to partition 0
    assert partition_batch(3, 3) == [(0, 1), (1, 1), (2, 1)]
    with pytest.raises(ValueError):
        partition_batch(2, 3)


def test_partition_by_proportions_follows_the_reference_rules():
    # the reference's own 4-GPU AlexNet placement: 0.25 each
    assert partition_by_proportions(256, [0.25] * 4) == [(i, 64 * i, 64) for i in range(4)]
    assert partition_by_proportions(2048, [0.125] * 8) == [(i, 256 * i, 256) for i in range(8)]
    # unequal shares; a GPU whose share truncates to zero is dropped
    assert partition_by_proportions(256, [0.5, 0.25, 0.25, 0.0]) == [(0, 0, 128), (1, 128, 64), (2, 192, 64)]
    # truncation leftovers: spread over the GPUs in use, the remainder to the first (3 x 85 = 255 of 256)
    assert partition_by_proportions(256, [1 / 3.0] * 3) == [(0, 0, 86), (1, 86, 85), (2, 171, 85)]
    assert partition_by_proportions(10, [0.75, 0.25]) == [(0, 0, 8), (1, 8, 2)]
    with pytest.raises(ValueError):
        partition_by_proportions(256, [0.25, 0.25])  # half the batch would go to CPU partitions: not built
    with pytest.raises(ValueError):
        partition_by_proportions(256, [0.75, 0.75])


def test_learning_rate_matches_oracle(port):
    for policy, args in (("fixed", (0.01, 0.1, 7.0, 3.0, 0.0, 1.0)), ("step", (0.01, 0.1, 7.0, 3.0, 0.0, 1.0)),
                         ("exp", (0.01, 0.9, 7.0, 3.0, 0.0, 1.0)), ("inv", (0.01, 0.1, 7.0, 3.0, 0.75, 1.0)),
                         ("poly", (0.01, 0.1, 7.0, 3.0, 2.0, 100.0)), ("sigmoid", (0.01, 0.1, 7.0, 3.0, 0.0, 1.0))):
        mine = get_learning_rate(policy, *args)
        theirs = port.learning_rate(policy, args[0], args[1], args[2], args[3], args[4], args[5])
        assert abs(mine - theirs) <= 1e-9 * max(1.0, abs(theirs)), policy


class HostCube:
    def __init__(self, arr):
        self.arr = arr
        self.ptr, self.n_elements, self.own_data = arr.ctypes.data, arr.size, True

    def free(self):
        self.arr = None


class HostOps:
    """numpy buffers + gloo all-reduce + the oracle's SGD step."""

    def __init__(self, port, world):
        self.port, self.world, self.keep = port, world, {}

    def alloc(self, count):
        a = np.zeros(count, np.float32)
        self.keep[a.ctypes.data] = a
        return a.ctypes.data

    def view(self, ptr, count):
        return np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_float)), shape=(count,))

    def zero(self, ptr, count):
        self.view(ptr, count)[:] = 0

    def allreduce_sum(self, ptr, count):
        if self.world > 1:
            import torch
            import torch.distributed as dist
            dist.all_reduce(torch.from_numpy(self.view(ptr, count)))

    def sgd_step(self, count, w, g, h, lr, momentum, lam, regularization_type="L2"):
        assert regularization_type == "L2"
        self.port.sgd_update(self.view(w, count), self.view(g, count), self.view(h, count), lr, momentum, lam)


class OracleSubBridge:
    """Stands in for the CUDA ConvolutionBridge of one rank: gradients of its batch slice from the oracle."""

    def __init__(self, port, ops, X, dY, W, b, k, s, p, g):
        self.port, self.ops, self.X, self.dY, self.geom = port, ops, X, dY, (k, s, p, g)
        self.bias_term = True
        self.w_shape = W.shape
        self.p_model_cube, self.p_bias_cube = HostCube(W.copy()), HostCube(b.copy())
        self.p_model_gradient_cube, self.p_bias_gradient_cube = HostCube(np.zeros_like(W)), HostCube(np.zeros_like(b))
        self.W0, self.b0 = W, b

    def _arr(self, cube):
        return self.ops.view(cube.ptr, cube.n_elements)

    def load_initial_model(self):
        self._arr(self.p_model_cube)[:] = self.W0.ravel()
        self._arr(self.p_bias_cube)[:] = self.b0

    def forward(self):
        pass

    def backward(self):
        k, s, p, g = self.geom
        W = self._arr(self.p_model_cube).reshape(self.w_shape).copy()
        _, dW, db = self.port.conv_backward(self.X, W, self.dY, k, s, p, g, needs_dx=False)
        self._arr(self.p_model_gradient_cube)[:] = dW.ravel()
        self._arr(self.p_bias_gradient_cube)[:] = db


def _rank_main(rank, world, port_file, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port_file), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    from oracle import pyoracle
    dist.init_process_group("gloo", rank=rank, world_size=world)
    port = pyoracle.port()
    B, D, n, o, k, s, p, g = SHAPE
    X, W, b, dY = make_inputs(77, B, D, n, o, k, s, p, g)
    start, size = partition_batch(B, world)[rank]
    ops = HostOps(port, world)
    sub = OracleSubBridge(port, ops, X[start:start + size].copy(), dY[start:start + size].copy(), W, b, k, s, p, g)
    pb = ParallelizedBridge(sub, SolverParameter(LR, "step", 0.1, 100000, momentum=MOM, weight_decay=WD), ops)
    sub.load_initial_model()
    for _ in range(2):
        pb.forward()
        pb.backward()
    np.save(os.path.join(out_dir, "params_%d.npy" % rank), ops.view(pb.params, pb.count).copy())
    dist.destroy_process_group()


def test_two_gloo_ranks_sum_gradients_and_step_like_one_process(port, tmp_path):
    import socket

    import torch.multiprocessing as mp
    with socket.socket() as sck:
        sck.bind(("127.0.0.1", 0))
        free_port = sck.getsockname()[1]
    mp.spawn(_rank_main, args=(2, free_port, str(tmp_path)), nprocs=2, join=True)
    p0, p1 = (np.load(os.path.join(str(tmp_path), "params_%d.npy" % r)) for r in (0, 1))
    assert np.array_equal(p0, p1)  # every rank applied the same update
    # one process, whole batch: two SGD steps with the oracle (weights lr_mult 1 / decay 1, bias lr_mult 2 / decay 0)
    B, D, n, o, k, s, p, g = SHAPE
    X, W, b, dY = make_inputs(77, B, D, n, o, k, s, p, g)
    W, b = W.copy(), b.copy()
    hw, hb = np.zeros_like(W), np.zeros_like(b)
    for it in (1, 2):
        _, dW, db = port.conv_backward(X, W, dY, k, s, p, g, needs_dx=False)
        lr = port.learning_rate("step", LR, 0.1, float(it), 100000.0)
        port.sgd_update(W, dW, hw, lr, MOM, WD)
        port.sgd_update(b, db, hb, float(np.float32(lr * 2.0)), MOM, 0.0)
    assert maxnorm_rel(p0[:W.size], W.ravel()) <= 1e-5
    assert maxnorm_rel(p0[W.size:], b) <= 1e-5


def test_against_reference_parallelized_bridge_with_two_partitions(port, reference):
    """The reference's own ParallelizedBridge (2 CPU partitions, SGD lr 0.01, no momentum) on the same inputs."""
    B, D, n, o, k, s, p, g = SHAPE
    X, W, b, dY = make_inputs(78, B, D, n, o, k, s, p, g)
    _, _, _, _, Wref, bref = reference.conv_fwd_bwd(X, W, b, dY, k, s, p, g=g, partitions=2, sgd=(LR, 0.0, 0.0))
    ops = HostOps(port, 1)
    grads = []
    for start, size in partition_batch(B, 2):
        _, dW, db = port.conv_backward(X[start:start + size].copy(), W, dY[start:start + size].copy(), k, s, p, g,
                                       needs_dx=False)
        grads.append((dW, db))
    sub = OracleSubBridge(port, ops, X, dY, W, b, k, s, p, g)
    pb = ParallelizedBridge(sub, SolverParameter(LR, "step", 0.1, 100000, momentum=0.0, weight_decay=0.0), ops,
                            lr_mult=(1.0, 1.0), decay_mult=(1.0, 1.0))
    sub.load_initial_model()
    sub.backward = lambda: (ops.view(pb.grads, pb.count).__setitem__(
        slice(None), np.concatenate([(grads[0][0] + grads[1][0]).ravel(), grads[0][1] + grads[1][1]])))
    pb.backward()
    mine = ops.view(pb.params, pb.count)
    assert maxnorm_rel(mine[:W.size], Wref.ravel()) <= 1e-5
    assert maxnorm_rel(mine[W.size:], bref) <= 1e-5
