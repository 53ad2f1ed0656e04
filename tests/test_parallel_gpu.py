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


def _run_rank(rank, world, device, steps, unique_id=None, proportions=None):
    """One rank's partition.  With `unique_id` the gradient sum goes through the library's own NCCL communicator
    (cct_comm_*), else through torch.distributed on torch's stream."""
    from caffecontroll_b200 import Context, ConvolutionBridge, Layer, LogicalCube
    from caffecontroll_b200.parallel import Communicator, DeviceOps, ParallelizedBridge, SolverParameter, partition_batch
    B, D, n, o, k, s, p, g = SHAPE
    m = (n + 2 * p - k) // s + 1
    X, W, b, dY = make_inputs(91, B, D, n, o, k, s, p, g)
    if proportions is None:
        start, size = partition_batch(B, world)[rank]
    else:  # unequal shares, as the reference's gpu_N_batch_proportion fields give them
        from caffecontroll_b200.parallel import partition_by_proportions
        _, start, size = partition_by_proportions(B, proportions)[rank]
    stream = None
    if world > 1 and unique_id is None:
        import torch
        torch.cuda.set_device(device)
        stream = torch.cuda.current_stream().cuda_stream
    ctx = Context(device, stream=stream)
    comm = Communicator(ctx, world, rank, unique_id) if unique_id is not None else None
    xin = Layer(LogicalCube.from_numpy(ctx, X[start:start + size]), LogicalCube(ctx, n, n, D, size))
    out = Layer(LogicalCube(ctx, m, m, o, size), LogicalCube.from_numpy(ctx, dY[start:start + size]))
    br = ConvolutionBridge(xin, out, k, s, p, g, True)
    br.needs_to_calc_backward_grad = False
    pb = ParallelizedBridge(br, SolverParameter(LR, "step", 0.1, 100000, momentum=MOM, weight_decay=WD),
                            DeviceOps(ctx, comm=comm))
    br.p_model_cube.upload(W)
    br.p_bias_cube.upload(b)
    for _ in range(steps):
        pb.forward()
        pb.backward()
    ctx.sync()
    res = br.p_model_cube.download(), br.p_bias_cube.download().ravel()
    if comm is not None:
        comm.close()
    return res


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


def _comm_rank(rank, world, id_path, out_dir):
    """No torch.distributed at all: rank 0 writes the NCCL id to a file, the others read it."""
    import time
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from caffecontroll_b200.parallel import Communicator
    if rank == 0:
        uid = Communicator.unique_id()
        with open(id_path + ".tmp", "wb") as f:
            f.write(uid)
        os.replace(id_path + ".tmp", id_path)
    else:
        for _ in range(600):
            if os.path.exists(id_path):
                break
            time.sleep(0.05)
        with open(id_path, "rb") as f:
            uid = f.read()
    W, b = _run_rank(rank, world, rank, 2, unique_id=uid, proportions=[0.75, 0.25])  # 6 + 2 of the 8 images
    np.save(os.path.join(out_dir, "W_%d.npy" % rank), W)
    np.save(os.path.join(out_dir, "b_%d.npy" % rank), b)


def test_two_ranks_through_the_c_abi_communicator_match_oracle(port, tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_comm_rank, args=(2, os.path.join(str(tmp_path), "nccl_id"), str(tmp_path)), nprocs=2, join=True)
    We, be = _expected(port, 2)
    W0, W1 = (np.load(os.path.join(str(tmp_path), "W_%d.npy" % r)) for r in (0, 1))
    b0 = np.load(os.path.join(str(tmp_path), "b_0.npy"))
    assert np.array_equal(W0, W1)
    assert maxnorm_rel(W0, We) <= TOL and maxnorm_rel(b0, be) <= TOL


def test_single_rank_communicator_is_a_no_op(ctx):
    from caffecontroll_b200.parallel import Communicator, DeviceOps
    comm = Communicator(ctx, 1, 0, None)
    ops = DeviceOps(ctx, comm=comm)
    buf = ops.alloc(16)
    ctx.fill(buf, 16, 3.0)
    ops.allreduce_sum(buf, 16)
    ctx.sync()
    out = np.empty(16, np.float32)
    ctx.d2h(out, buf)
    assert np.all(out == 3.0)
    ops.free(buf)
    comm.close()
