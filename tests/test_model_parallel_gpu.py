"""Model-parallel fully connected layers (the split -> per-GPU slices -> concat construction of src/DeepNet.h:1213-1357):
one rank against the plain bridge, two NCCL ranks against a float64 product over the whole mini-batch, and a
prototxt-built net with its fc6 / fc7 split over two ranks against the same net run data parallel."""
import os
import sys
import time

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from tests.parity import TOL, maxnorm_rel  # noqa: E402

pytestmark = pytest.mark.gpu
B_LOCAL, D, N, OUT = 40, 6, 4, 72  # per-rank batch, input cube D x N x N, outputs


def _problem(world):
    rng = np.random.default_rng(77)
    Bg, K = B_LOCAL * world, D * N * N
    X = rng.standard_normal((Bg, D, N, N), dtype=np.float32)
    W = (0.1 * rng.standard_normal((OUT, K))).astype(np.float32)
    b = rng.standard_normal(OUT, dtype=np.float32)
    dY = rng.standard_normal((Bg, OUT, 1, 1), dtype=np.float32)
    return X, W, b, dY


def _expected(world):
    X, W, b, dY = _problem(world)
    x, g = X.reshape(X.shape[0], -1).astype(np.float64), dY.reshape(dY.shape[0], -1).astype(np.float64)
    return x @ W.T.astype(np.float64) + b, g @ W.astype(np.float64), g.T @ x, g.sum(0)


def _run_bridge(ctx, comm, world, rank):
    from caffecontroll_b200 import Layer, LogicalCube
    from caffecontroll_b200.parallel import ModelParallelFullyConnectedBridge
    X, W, b, dY = _problem(world)
    rows = slice(rank * B_LOCAL, (rank + 1) * B_LOCAL)
    xin = Layer(LogicalCube.from_numpy(ctx, X[rows]), LogicalCube(ctx, N, N, D, B_LOCAL))
    out = Layer(LogicalCube(ctx, 1, 1, OUT, B_LOCAL), LogicalCube.from_numpy(ctx, dY[rows]))
    br = ModelParallelFullyConnectedBridge(xin, out, comm)
    br.set_model_host(W, b)
    br.forward()
    br.backward()
    ctx.sync()
    res = dict(Y=out.p_data_cube.download().reshape(B_LOCAL, OUT), dX=xin.p_gradient_cube.download().reshape(B_LOCAL, -1),
               dW=br.p_model_gradient_cube.download().reshape(br.slice_depth, -1),
               db=br.p_bias_gradient_cube.download().ravel())
    w_all, b_all = br.model_host()  # the gathered matrix is the one that was handed in
    assert np.array_equal(w_all.reshape(OUT, -1), W) and np.array_equal(b_all.ravel(), b)
    br.close()
    return res


def _check(res, world, rank):
    Y, dX, dW, db = _expected(world)
    rows = slice(rank * B_LOCAL, (rank + 1) * B_LOCAL)
    cols = slice(rank * (OUT // world), (rank + 1) * (OUT // world))
    errs = dict(Y=maxnorm_rel(res["Y"], Y[rows]), dX=maxnorm_rel(res["dX"], dX[rows]),
                dW=maxnorm_rel(res["dW"], dW[cols]), db=maxnorm_rel(res["db"], db[cols]))
    assert max(errs.values()) <= TOL, errs


def test_one_rank_equals_the_plain_bridge(ctx):
    from caffecontroll_b200 import FullyConnectedBridge, Layer, LogicalCube
    from caffecontroll_b200.parallel import Communicator
    comm = Communicator(ctx, 1, 0, None)
    res = _run_bridge(ctx, comm, 1, 0)
    _check(res, 1, 0)
    X, W, b, dY = _problem(1)
    xin = Layer(LogicalCube.from_numpy(ctx, X), LogicalCube(ctx, N, N, D, B_LOCAL))
    out = Layer(LogicalCube(ctx, 1, 1, OUT, B_LOCAL), LogicalCube.from_numpy(ctx, dY))
    br = FullyConnectedBridge(xin, out)
    br.p_model_cube.upload(W.reshape(br.p_model_cube.shape))
    br.p_bias_cube.upload(b.reshape(br.p_bias_cube.shape))
    br.forward()
    br.backward()
    ctx.sync()
    assert np.array_equal(out.p_data_cube.download().reshape(B_LOCAL, OUT), res["Y"])
    assert np.array_equal(xin.p_gradient_cube.download().reshape(B_LOCAL, -1), res["dX"])
    assert np.array_equal(br.p_model_gradient_cube.download().reshape(OUT, -1), res["dW"])
    br.close()
    comm.close()


def _rank_main(rank, world, id_path, out_dir):
    """No torch.distributed: rank 0 writes the NCCL id to a file, the others read it."""
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from caffecontroll_b200 import Context
    from caffecontroll_b200.net import Net, parse_prototxt, solver_from_message
    from caffecontroll_b200.parallel import Communicator, DeviceOps
    from tests.test_net_gpu import NET, SOLVER
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
    ctx = Context(rank)
    comm = Communicator(ctx, world, rank, uid)
    _check(_run_bridge(ctx, comm, world, rank), world, rank)

    # the same net data parallel and with fc6 / fc7 split over the ranks: same parameters at the start (the slices are
    # cut from the whole layer's filler output), same losses, same updates
    Bn = 8
    rng = np.random.default_rng(123)
    X = rng.standard_normal((Bn * world, 3, 67, 67), dtype=np.float32)
    labels = rng.integers(0, 12, Bn * world).astype(np.float32)
    rows = slice(rank * Bn, (rank + 1) * Bn)
    out = {}
    for tag, names in (("dp", ()), ("mp", ("fc6", "fc7"))):
        net = Net(ctx, parse_prototxt(NET), solver_from_message(parse_prototxt(SOLVER)), Bn, ops=DeviceOps(ctx, comm=comm),
                  loss_batch=Bn * world, model_parallel=names)
        net.set_input(X[rows], labels[rows])
        path = os.path.join(out_dir, "%s_%d" % (tag, rank))
        net.write_model_to_file(path + ".init")
        losses = []
        for _ in range(2):
            net.step()
            losses.append(net.get_loss())
        net.write_snapshot(path)
        out[tag] = losses
        if tag == "mp":  # a snapshot read back into the split layers restores every slice
            net.step()
            net.read_snapshot(path)
            net.write_snapshot(path + "_again")
        net.close()
    np.save(os.path.join(out_dir, "loss_%d.npy" % rank), np.array([out["dp"], out["mp"]], np.float64))
    comm.close()


def test_two_ranks_match_the_whole_batch_product_and_the_data_parallel_net(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    d = str(tmp_path)
    mp.spawn(_rank_main, args=(2, os.path.join(d, "nccl_id"), d), nprocs=2, join=True)
    load = lambda name: np.fromfile(os.path.join(d, name), np.float32)
    for r in (0, 1):
        assert np.array_equal(load("mp_%d.init" % r), load("dp_0.init"))  # gathered slices = the whole layer's fill
        for ext in (".MODEL", ".HISTORY"):
            dp, mpar, init = load("dp_0" + ext), load("mp_%d" % r + ext), load("dp_0.init")
            base = init if ext == ".MODEL" else np.zeros_like(dp)
            assert maxnorm_rel(mpar - base, dp - base) <= 1e-3, (r, ext)
            assert np.array_equal(load("mp_%d_again" % r + ext), mpar), (r, ext)
        loss = np.load(os.path.join(d, "loss_%d.npy" % r))
        assert np.allclose(loss[0], loss[1], rtol=1e-5), loss
