"""GPU tests of the ParallelizedBridge mirror driving the CUDA convolution bridge: one rank always, two NCCL ranks
where the box has two GPUs.  Expected values come from the CPU oracle run on the whole batch."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from tests.parity import TOL, make_inputs, maxnorm_rel  # noqa: E402

pytestmark = pytest.mark.gpu
SHAPE = (8, 6, 13, 10, 3, 1, 1, 1)  # B, D, n, o, k, s, p, g
LR, MOM, WD = 0.01, 0.9, 0.0005


def _expected(port, steps):
    B, D, n, o, k, s, p, g = SHAPE
    X, W, b, dY = make_inputs(91, B, D, n, o, k, s, p, g)
    W, b = W.copy(), b.copy()
    hw, hb = np.zeros_like(W), np.zeros_like(b)
    for it in range(1, steps + 1):
        _, dW, db = port.conv_backward(X, W, dY, k, s, p, g, needs_dx=False)
        lr = port.learning_rate("step", LR, 0.1, float(it), 100000.0)
        port.sgd_update(W, dW, hw, lr, MOM, WD)
        port.sgd_update(b, db, hb, float(np.float32(lr * 2.0)), MOM, 0.0)
    return W, b


def _run_rank(rank, world, device, steps):
    from caffecontroll_b200 import Context, ConvolutionBridge, Layer, LogicalCube
    from caffecontroll_b200.parallel import DeviceOps, ParallelizedBridge, SolverParameter, partition_batch
    B, D, n, o, k, s, p, g = SHAPE
    m = (n + 2 * p - k) // s + 1
    X, W, b, dY = make_inputs(91, B, D, n, o, k, s, p, g)
    start, size = partition_batch(B, world)[rank]
    stream = None
    if world > 1:
        import torch
        torch.cuda.set_device(device)
        stream = torch.cuda.current_stream().cuda_stream
    ctx = Context(device, stream=stream)
    xin = Layer(LogicalCube.from_numpy(ctx, X[start:start + size]), LogicalCube(ctx, n, n, D, size))
    out = Layer(LogicalCube(ctx, m, m, o, size), LogicalCube.from_numpy(ctx, dY[start:start + size]))
    br = ConvolutionBridge(xin, out, k, s, p, g, True)
    br.needs_to_calc_backward_grad = False
    pb = ParallelizedBridge(br, SolverParameter(LR, "step", 0.1, 100000, momentum=MOM, weight_decay=WD), DeviceOps(ctx))
    br.p_model_cube.upload(W)
    br.p_bias_cube.upload(b)
    for _ in range(steps):
        pb.forward()
        pb.backward()
    ctx.sync()
    return br.p_model_cube.download(), br.p_bias_cube.download().ravel()


def test_single_rank_step_matches_oracle(port):
    W, b = _run_rank(0, 1, 0, 2)
    We, be = _expected(port, 2)
    assert maxnorm_rel(W, We) <= TOL and maxnorm_rel(b, be) <= TOL


def _nccl_rank(rank, world, port_no, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port_no), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    W, b = _run_rank(rank, world, rank, 2)
    np.save(os.path.join(out_dir, "W_%d.npy" % rank), W)
    np.save(os.path.join(out_dir, "b_%d.npy" % rank), b)
    dist.barrier()
    dist.destroy_process_group()


def test_two_nccl_ranks_match_oracle_on_whole_batch(port, tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as sck:
        sck.bind(("127.0.0.1", 0))
        port_no = sck.getsockname()[1]
    mp.spawn(_nccl_rank, args=(2, port_no, str(tmp_path)), nprocs=2, join=True)
    We, be = _expected(port, 2)
    W0, W1 = (np.load(os.path.join(str(tmp_path), "W_%d.npy" % r)) for r in (0, 1))
    b0 = np.load(os.path.join(str(tmp_path), "b_0.npy"))
    assert np.array_equal(W0, W1)
    assert maxnorm_rel(W0, We) <= TOL and maxnorm_rel(b0, be) <= TOL
