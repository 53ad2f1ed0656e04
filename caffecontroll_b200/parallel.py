"""ParallelizedBridge's batch partitioning for one process per GPU.

The reference splits a layer's mini-batch into contiguous partitions, runs one sub-bridge per partition, SUMS the
partitions' model gradients on the host and applies one SGD step (src/bridges/ParallelizedBridge.h:615-719,
src/bridges/ParallelizedBridge_impl.hxx:761-1065).  Here every rank owns one partition and one sub-bridge; parameters,
gradients and momentum history live in one flat device buffer per rank (W | bias), the gradient sum is one all-reduce
over that buffer (NCCL through torch.distributed), and every rank applies the same update, so no broadcast is needed.

The arithmetic that touches a device sits behind a small `ops` object so the host logic (slicing, iteration counter,
learning-rate policy, per-blob multipliers) can be exercised with gloo ranks on CPU.
"""
import ctypes as C
import math

import numpy as np

from . import capi


def partition_batch(global_batch, n_partitions):
    """Contiguous slices [(start, size)] of the mini-batch, one per partition: equal shares by truncation, the
    remainder goes to partition 0 (as the reference gives leftovers to GPU 0, ParallelizedBridge.h:690-719)."""
    if n_partitions <= 0 or global_batch < n_partitions:
        raise ValueError("need 1 <= n_partitions <= global_batch")
    share = global_batch // n_partitions
    sizes = [share] * n_partitions
    sizes[0] += global_batch - share * n_partitions
    out, start = [], 0
    for s in sizes:
        out.append((start, s))
        start += s
    return out


def partition_by_proportions(global_batch, proportions):
    """GPU batch sizes from per-GPU batch proportions, the reference's placement fields gpu_{0..3}_batch_proportion
    (src/parser/cnn.proto:249-256; any number of GPUs here).  As ParallelizedBridge::update_scheduler_partitions_for_curr_B
    does (src/bridges/ParallelizedBridge.h:615-719): GPU i takes trunc(proportion_i * batch) images, GPUs whose share
    comes out as zero are dropped, and the images left over by the truncation are spread over the GPUs in use, the
    remainder of that division going to the first one.  Returns [(gpu index, start, size)] with contiguous slices in
    GPU order.  The reference hands whatever the proportions do not cover to CPU partitions; there is no CPU path here,
    so proportions that leave more than the truncation's leftovers uncovered are refused."""
    if global_batch <= 0 or not proportions or any(p < 0 for p in proportions):
        raise ValueError("need a positive batch and non-negative proportions")
    sizes = [(i, int(p * global_batch)) for i, p in enumerate(proportions)]
    sizes = [(i, n) for i, n in sizes if n > 0]
    if not sizes:
        raise ValueError("no GPU receives any image")
    left = global_batch - sum(n for _, n in sizes)
    if left < 0:
        raise ValueError("proportions add up to more than the batch")
    if left >= len(proportions) + 1 and sum(proportions) < 1.0 - 1e-6:
        raise ValueError("proportions leave %d of %d images to CPU partitions, which are not built (no CPU fallback)" %
                         (left, global_batch))
    per, extra = left // len(sizes), left % len(sizes)
    out, start = [], 0
    for j, (i, n) in enumerate(sizes):
        n += per + (extra if j == 0 else 0)
        out.append((i, start, n))
        start += n
    return out


class SolverParameter:
    """The solver fields the updater reads (src/algorithms/GradientUpdater.h:60-120, src/util.h:76-100)."""

    def __init__(self, base_lr=0.01, lr_policy="step", gamma=0.1, stepsize=100000, power=0.0, max_iter=1, momentum=0.9,
                 weight_decay=0.0005, regularization_type="L2"):
        self.base_lr, self.lr_policy, self.gamma, self.stepsize = base_lr, lr_policy, gamma, stepsize
        self.power, self.max_iter, self.momentum, self.weight_decay = power, max_iter, momentum, weight_decay
        self.regularization_type = regularization_type


def get_learning_rate(policy, base_lr, gamma, it, stepsize, power, max_iter):
    """Util::get_learning_rate (src/util.h:76-100), evaluated in double and rounded to float like the reference."""
    if policy == "fixed":
        rate = base_lr
    elif policy == "step":
        rate = base_lr * math.pow(gamma, int(it / stepsize))
    elif policy == "exp":
        rate = base_lr * math.pow(gamma, it)
    elif policy == "inv":
        rate = base_lr * math.pow(1.0 + gamma * it, -power)
    elif policy == "poly":
        rate = base_lr * math.pow(1.0 - it / max_iter, power)
    elif policy == "sigmoid":
        rate = base_lr * (1.0 / (1.0 + math.exp(-gamma * (it - stepsize))))
    else:
        raise ValueError("unknown lr_policy %r" % policy)
    return float(np.float32(rate))


class Communicator:
    """cct_comm: the NCCL communicator of the C ABI (one per context).  `unique_id` is the 128-byte id rank 0 made with
    Communicator.unique_id() and handed to every rank; nranks == 1 needs none and never loads NCCL."""

    def __init__(self, ctx, nranks=1, rank=0, unique_id=None):
        self.ctx, self.nranks, self.rank = ctx, nranks, rank
        h = C.c_void_p()
        capi.check(ctx.lib.cct_comm_init_rank(ctx.h, nranks, rank, unique_id, C.byref(h)), "cct_comm_init_rank", ctx.h)
        self.h = h

    @staticmethod
    def unique_id():
        buf = C.create_string_buffer(capi.COMM_ID_BYTES)
        capi.check(capi.load().cct_comm_unique_id(buf), "cct_comm_unique_id")
        return buf.raw

    def allgather(self, send_ptr, recv_ptr, count_per_rank):
        """recv[r * count_per_rank ...] = rank r's block of count_per_rank floats, on every rank."""
        capi.check(self.ctx.lib.cct_allgather(self.h, C.c_void_p(send_ptr), C.c_void_p(recv_ptr), count_per_rank),
                   "cct_allgather", self.ctx.h)

    def reduce_scatter_sum(self, send_ptr, recv_ptr, count_per_rank):
        """recv = the sum over ranks of their send[rank * count_per_rank ...] blocks."""
        capi.check(self.ctx.lib.cct_reduce_scatter_sum(self.h, C.c_void_p(send_ptr), C.c_void_p(recv_ptr), count_per_rank),
                   "cct_reduce_scatter_sum", self.ctx.h)

    def close(self):
        if self.h:
            self.ctx.lib.cct_comm_destroy(self.h)
            self.h = None


def model_parallel_gpus(depth_proportions, output_depth):
    """The GPUs of a model-parallel layer from its placement fields gpu_{0..3}_depth_proportion, with the checks of
    DeepNet::get_model_parallelism_info (src/DeepNet.h:728-790): every share divides the output depth exactly, all
    non-zero shares are equal, they add up to 1 over two or more GPUs - or are all zero (no model parallelism: [])."""
    used, share = [], 0.0
    for i, p in enumerate(depth_proportions):
        if p == 1.0:
            raise ValueError("a depth proportion of 1.0: model parallelism needs two or more GPUs (use batch proportions)")
        if p < 0 or float(output_depth) * p != int(float(output_depth) * p):
            raise ValueError("model parallelism must divide the output depth exactly (depth %d, proportion %g)" %
                             (output_depth, p))
        if p > 0:
            if share and p != share:
                raise ValueError("every GPU of a model-parallel layer must have the same depth proportion")
            share = p
            used.append(i)
    total = sum(depth_proportions)
    if not used:
        return []
    if abs(total - 1.0) > 1e-6:
        raise ValueError("depth proportions must add up to 1 (model parallelism is all on the GPUs)")
    return used


class DeviceOps:
    """Gradient sum and SGD step on the GPU.  The sum is an NCCL all-reduce issued through the C ABI's communicator
    (on its own stream, overlapping the kernels queued after it) when one is given, else through torch.distributed on
    torch's current stream - which must then be the stream the context was created on."""

    def __init__(self, ctx, group=None, comm=None):
        self.ctx, self.group, self.comm = ctx, group, comm
        self._checked_stream = False

    def world_size(self):
        if self.comm is not None:
            return self.comm.nranks
        import torch.distributed as dist
        return dist.get_world_size(self.group) if dist.is_available() and dist.is_initialized() else 1

    def alloc(self, count):
        return self.ctx.malloc(4 * count)

    def free(self, ptr):
        self.ctx.free(ptr)

    def view(self, ptr, count):
        import torch

        class _Iface:  # zero-copy: torch wraps the pointer through the CUDA array interface
            __cuda_array_interface__ = {"shape": (count,), "typestr": "<f4", "data": (ptr, False), "version": 3}

        return torch.as_tensor(_Iface(), device="cuda:%d" % self.ctx.device)

    def allreduce_begin(self, ptr, count):
        """Starts the sum of `count` floats at `ptr` over all ranks, ordered behind the work queued so far."""
        if self.comm is not None:
            capi.check(self.ctx.lib.cct_allreduce_sum_begin(self.comm.h, C.c_void_p(ptr), count), "cct_allreduce_sum_begin",
                       self.ctx.h)
        elif self.world_size() > 1:
            import torch
            import torch.distributed as dist
            if not self._checked_stream:
                # the collective runs on torch's current stream; the kernels that produce and consume the buffer run on
                # the context's stream: without a communicator of its own the two must be one stream
                cur = torch.cuda.current_stream(self.ctx.device).cuda_stream
                if self.ctx.stream != cur:
                    raise RuntimeError("DeviceOps without a Communicator needs a Context created on torch's current "
                                       "stream (Context(device, stream=torch.cuda.current_stream().cuda_stream))")
                self._checked_stream = True
            dist.all_reduce(self.view(ptr, count), group=self.group)

    def allreduce_wait(self):
        """Orders the context's stream behind every sum begun so far."""
        if self.comm is not None:
            capi.check(self.ctx.lib.cct_comm_wait(self.comm.h), "cct_comm_wait", self.ctx.h)

    def allreduce_sum(self, ptr, count):
        self.allreduce_begin(ptr, count)
        self.allreduce_wait()

    def sgd_step(self, count, w, g, h, lr, momentum, lam, regularization_type="L2"):
        """SGDGradientUpdater::update (src/algorithms/GradientUpdater.h:154-193): "L2" adds lam * w to the gradient,
        "L1" lam * sign(w) (DeviceDriver::L1_update), then the momentum step; any other type applies no decay, as there."""
        vp = C.c_void_p
        if lam != 0.0 and regularization_type == "L1":
            capi.check(self.ctx.lib.cct_l1_update(self.ctx.h, count, vp(g), lam, vp(w)), "cct_l1_update", self.ctx.h)
        if regularization_type != "L2":
            lam = 0.0
        capi.check(self.ctx.lib.cct_sgd_step(self.ctx.h, count, vp(w), vp(g), vp(h), lr, momentum, lam), "cct_sgd_step",
                   self.ctx.h)

    def zero(self, ptr, count):
        self.ctx.fill(ptr, count, 0.0)

    def copy(self, dst, src, count):
        capi.check(self.ctx.lib.cct_memcpy_d2d(self.ctx.h, C.c_void_p(dst), C.c_void_p(src), 4 * count), "cct_memcpy_d2d",
                   self.ctx.h)
        self.ctx.sync()  # the source is freed right after


class SliceOps(DeviceOps):
    """DeviceOps for parameters that only this rank holds (a slice of a model-parallel layer): its gradients are already
    those of the whole mini-batch, so there is nothing to sum."""

    def __init__(self, ctx):
        super().__init__(ctx, comm=None)

    def world_size(self):
        return 1

    def allreduce_begin(self, ptr, count):
        pass

    def allreduce_wait(self):
        pass


class ModelParallelFullyConnectedBridge:
    """A fully connected layer split over the ranks by output depth: what DeepNet builds as split bridge -> one
    FullyConnectedBridge per GPU over output_depth / n_gpus outputs, each on the whole mini-batch -> concat bridge
    (src/DeepNet.h:1213-1357), with the host round trips of those two bridges replaced by NCCL exchanges.

    The layers around it stay data parallel, so its input and output layers hold this rank's batch slice:
      forward   all-gather of the input slices (every rank sees the whole mini-batch, as behind the reference's split
                bridge) -> this rank's output slice for the whole batch -> all-gather of the slices, of which the rows of
                this rank's images are copied side by side into its output cube (the concat bridge);
      backward  all-gather of the output gradients, this rank's columns of it -> weight / bias gradient of the slice (over
                the whole mini-batch: no gradient sum is needed) and its share of the input gradient for every image ->
                reduce-scatter: each rank receives the sum over the slices for its own images (SplitBridge::backward,
                src/bridges/SplitBridge_impl.hxx:51-90).
    Model and bias cubes are this rank's slice (rows rank * O / n ... of the [num_output][in_features] matrix)."""

    algo = capi.ALGO_SIMT_FP32  # keeps the network's fusion pass away: the ReLU / dropout bridges around it run as bridges
    plan = None                 # the plan belongs to the inner bridge

    def __init__(self, p_input_layer, p_output_layer, comm, bias_term=True, algo=capi.ALGO_AUTO, ctx=None):
        from .bridge import FullyConnectedBridge, Layer, LogicalCube
        x, y = p_input_layer.p_data_cube, p_output_layer.p_data_cube
        self.p_input_layer, self.p_output_layer = p_input_layer, p_output_layer
        self.ctx = ctx or x.ctx
        self.lib, self.comm = self.ctx.lib, comm
        self.world, self.rank = comm.nranks, comm.rank
        self.iR, self.iC, self.iD, self.iB = x.R, x.C, x.D, x.B
        self.oR, self.oC, self.oD, self.oB = y.R, y.C, y.D, y.B
        if (self.oR, self.oC, self.oB) != (1, 1, self.iB):
            raise ValueError("output layer must be B x num_output x 1 x 1")
        if self.oD % self.world:
            raise ValueError("model parallelism must divide the output depth exactly (%d outputs, %d GPUs)" %
                             (self.oD, self.world))
        self.slice_depth = self.oD // self.world
        self.in_features = x.D * x.R * x.C
        self.global_batch = self.iB * self.world
        self.bias_term = bias_term
        self.needs_to_calc_backward_grad = True
        c, Bg = self.ctx, self.global_batch
        self.all_in = Layer(LogicalCube(c, x.R, x.C, x.D, Bg), LogicalCube(c, x.R, x.C, x.D, Bg))
        self.slice_out = Layer(LogicalCube(c, 1, 1, self.slice_depth, Bg), LogicalCube(c, 1, 1, self.slice_depth, Bg))
        self.staging = LogicalCube(c, 1, 1, self.oD, Bg)  # gathered output slices / gathered output gradients
        self.inner = FullyConnectedBridge(self.all_in, self.slice_out, bias_term, algo, c)
        i = self.inner
        self.p_model_cube, self.p_model_gradient_cube = i.p_model_cube, i.p_model_gradient_cube
        self.p_bias_cube, self.p_bias_gradient_cube = i.p_bias_cube, i.p_bias_gradient_cube

    def get_model_cube(self):
        return self.p_model_cube

    def get_bias_cube(self):
        return self.p_bias_cube

    def get_model_grad_cube(self):
        return self.p_model_gradient_cube

    def get_bias_grad_cube(self):
        return self.p_bias_gradient_cube

    def _copy2d(self, dst, dst_pitch, src, src_pitch, width, rows):
        capi.check(self.lib.cct_memcpy2d_d2d(self.ctx.h, C.c_void_p(dst), 4 * dst_pitch, C.c_void_p(src), 4 * src_pitch,
                                             4 * width, rows), "cct_memcpy2d_d2d", self.ctx.h)

    def forward(self):
        B, Bg, K, O, Os = self.iB, self.global_batch, self.in_features, self.oD, self.slice_depth
        self.comm.allgather(self.p_input_layer.p_data_cube.ptr, self.all_in.p_data_cube.ptr, B * K)
        self.inner.forward()
        self.comm.allgather(self.slice_out.p_data_cube.ptr, self.staging.ptr, Bg * Os)
        y = self.p_output_layer.p_data_cube.ptr
        for q in range(self.world):  # rank q's slice for this rank's images -> columns q * Os ... of the output cube
            self._copy2d(y + 4 * q * Os, O, self.staging.ptr + 4 * (q * Bg + self.rank * B) * Os, Os, Os, B)

    def backward(self):
        B, Bg, K, O, Os = self.iB, self.global_batch, self.in_features, self.oD, self.slice_depth
        self.comm.allgather(self.p_output_layer.p_gradient_cube.ptr, self.staging.ptr, B * O)
        self._copy2d(self.slice_out.p_gradient_cube.ptr, Os, self.staging.ptr + 4 * self.rank * Os, O, Os, Bg)
        self.inner.needs_to_calc_backward_grad = self.needs_to_calc_backward_grad
        self.inner.backward()
        if self.needs_to_calc_backward_grad:
            self.comm.reduce_scatter_sum(self.all_in.p_gradient_cube.ptr, self.p_input_layer.p_gradient_cube.ptr, B * K)

    # the whole layer's parameters to / from the host (every rank calls these: they gather over the ranks)
    def gather_host(self, ptr, n):
        """n floats at `ptr` of every rank, in rank order, as one host array (a collective: every rank calls it)."""
        from .bridge import LogicalCube
        full = LogicalCube(self.ctx, 1, 1, n, self.world)
        self.comm.allgather(ptr, full.ptr, n)
        self.ctx.sync()
        out = full.download().ravel()
        full.free()
        return out

    def model_host(self):
        w = self.gather_host(self.p_model_cube.ptr, self.p_model_cube.n_elements).reshape(self.oD, self.iD, self.iR, self.iC)
        b = self.gather_host(self.p_bias_cube.ptr, self.slice_depth).reshape(1, self.oD, 1, 1) if self.bias_term else None
        return w, b

    def set_model_host(self, w, b=None):
        Os = self.slice_depth
        w = np.ascontiguousarray(w, np.float32).reshape(self.oD, -1)
        self.p_model_cube.upload(w[self.rank * Os:(self.rank + 1) * Os].reshape(self.p_model_cube.shape))
        if self.bias_term and b is not None:
            b = np.ascontiguousarray(b, np.float32).ravel()
            self.p_bias_cube.upload(b[self.rank * Os:(self.rank + 1) * Os].reshape(self.p_bias_cube.shape))

    def close(self):
        self.inner.close()
        for layer in (self.all_in, self.slice_out):
            layer.p_data_cube.free()
            layer.p_gradient_cube.free()
        self.staging.free()


class ParallelizedBridge:
    """One rank's share of a data-parallel convolution layer.

    `bridge` is this rank's sub-bridge over its batch slice (a ConvolutionBridge).  Its model, bias and gradient cubes
    are re-pointed into one flat buffer owned here, as the reference's ParallelizedBridge owns p_model_cube and hands
    the pointer to its sub-bridges (ParallelizedBridge_impl.hxx:519-532).
    """

    def __init__(self, bridge, solver, ops, lr_mult=(1.0, 2.0), decay_mult=(1.0, 0.0), defer_update=False):
        self.bridge, self.solver, self.ops = bridge, solver, ops
        self.defer_update = defer_update  # backward() only begins the gradient sum; the owner calls apply_update()
        self.n_w = bridge.p_model_cube.n_elements
        self.n_b = bridge.p_bias_cube.n_elements if bridge.bias_term else 0
        n = self.n_w + self.n_b
        self.count = n
        self.params, self.grads, self.hist = ops.alloc(n), ops.alloc(n), ops.alloc(n)
        ops.zero(self.hist, n)
        # the sub-bridge's model and bias (already filled by its constructor's fillers) move into the flat buffer, as
        # the reference's ParallelizedBridge copies sub-bridge 0's model into its own cube (ParallelizedBridge_impl.hxx:130-160)
        copy = getattr(ops, "copy", None)
        if copy is not None:
            copy(self.params, bridge.p_model_cube.ptr, self.n_w)
            if self.n_b:
                copy(self.params + 4 * self.n_w, bridge.p_bias_cube.ptr, self.n_b)
        self._repoint(bridge.p_model_cube, self.params)
        self._repoint(bridge.p_model_gradient_cube, self.grads)
        if self.n_b:
            self._repoint(bridge.p_bias_cube, self.params + 4 * self.n_w)
            self._repoint(bridge.p_bias_gradient_cube, self.grads + 4 * self.n_w)
        self.lr_mult, self.decay_mult = lr_mult, decay_mult
        self.current_iter = 0
        self.update_model_gradients = True

    @staticmethod
    def _repoint(cube, ptr):
        cube.free()
        cube.ptr, cube.own_data = ptr, False

    # names of the reference's scheduler-facing interface
    def set_update_model_gradients(self, flag):
        self.update_model_gradients = flag

    def set_current_iter(self, it):
        self.current_iter = it

    def get_model_cube(self):
        return self.bridge.p_model_cube

    def get_bias_cube(self):
        return self.bridge.p_bias_cube

    def forward(self):
        self.bridge.forward()

    def backward(self, begin_allreduce=True):
        """The sub-bridge's backward pass, then the gradient sum is begun (not waited for).  A caller that wants the sum
        to start later - behind further kernels - passes begin_allreduce=False and calls begin_allreduce() itself."""
        self.bridge.backward()
        if not begin_allreduce and self.defer_update and hasattr(self.ops, "allreduce_begin"):
            return
        self.begin_allreduce()
        if not self.defer_update:
            wait = getattr(self.ops, "allreduce_wait", None)
            if hasattr(self.ops, "allreduce_begin") and wait is not None:
                wait()
            self.apply_update()

    def begin_allreduce(self):
        begin = getattr(self.ops, "allreduce_begin", None)
        if begin is None:  # an ops object with the blocking form only
            self.ops.allreduce_sum(self.grads, self.count)
        else:
            begin(self.grads, self.count)  # gradients are summed, not averaged (:916-955)

    def apply_update(self):
        """The SGD step on the summed gradients (the caller has waited for the sum when updates are deferred)."""
        if not self.update_model_gradients:
            return
        s = self.solver
        self.current_iter += 1  # the updater increments before use (GradientUpdater.h:155)
        base = get_learning_rate(s.lr_policy, s.base_lr, s.gamma, float(self.current_iter), float(s.stepsize), s.power,
                                 float(s.max_iter))
        self.ops.sgd_step(self.n_w, self.params, self.grads, self.hist, float(np.float32(base * self.lr_mult[0])),
                          s.momentum, float(np.float32(s.weight_decay * self.decay_mult[0])), s.regularization_type)
        if self.n_b:
            off = 4 * self.n_w
            self.ops.sgd_step(self.n_b, self.params + off, self.grads + off, self.hist + off,
                              float(np.float32(base * self.lr_mult[1])), s.momentum,
                              float(np.float32(s.weight_decay * self.decay_mult[1])), s.regularization_type)

    def get_model_grad_cube(self):
        return self.bridge.p_model_gradient_cube

    # momentum history to / from the host (force_device_to_host_*_history_copy, src/bridges/ParallelizedBridge.h:482-507)
    def history_host(self):
        ctx = self.bridge.ctx
        ctx.sync()
        h = np.empty(self.count, np.float32)
        ctx.d2h(h, self.hist)
        return h[:self.n_w].copy(), (h[self.n_w:].copy() if self.n_b else None)

    def set_history_host(self, w_hist, b_hist=None):
        ctx = self.bridge.ctx
        h = np.concatenate([np.ascontiguousarray(w_hist, np.float32).ravel()] +
                           ([np.ascontiguousarray(b_hist, np.float32).ravel()] if self.n_b else []))
        ctx.h2d(self.hist, h)

    def get_bias_grad_cube(self):
        return self.bridge.p_bias_gradient_cube

    def close(self):
        free = getattr(self.ops, "free", None)
        if free is not None:
            for p in (self.params, self.grads, self.hist):
                free(p)
        self.params = self.grads = self.hist = None


class ModelParallelizedBridge(ParallelizedBridge):
    """The updater around a ModelParallelFullyConnectedBridge: this rank's slice of the parameters, their gradients over
    the whole mini-batch (so no sum over ranks) and their momentum history.  The host-side views (model files,
    snapshots) are those of the whole layer: reading gathers the slices in rank order - the rows of the
    [num_output][in_features] matrix in order - and is a collective every rank takes part in."""

    def __init__(self, bridge, solver, ctx, lr_mult=(1.0, 2.0), decay_mult=(1.0, 0.0), defer_update=False):
        super().__init__(bridge, solver, SliceOps(ctx), lr_mult, decay_mult, defer_update)

    def model_host(self):
        return self.bridge.model_host()

    def set_model_host(self, w, b=None):
        self.bridge.set_model_host(w, b)

    @property
    def full_counts(self):
        return self.n_w * self.bridge.world, self.n_b * self.bridge.world

    def history_host(self):
        w = self.bridge.gather_host(self.hist, self.n_w)
        b = self.bridge.gather_host(self.hist + 4 * self.n_w, self.n_b) if self.n_b else None
        return w, b

    def set_history_host(self, w_hist, b_hist=None):
        r = self.bridge.rank
        w = np.ascontiguousarray(w_hist, np.float32).ravel()[r * self.n_w:(r + 1) * self.n_w]
        b = np.ascontiguousarray(b_hist, np.float32).ravel()[r * self.n_b:(r + 1) * self.n_b] if self.n_b else None
        super().set_history_host(w, b)

