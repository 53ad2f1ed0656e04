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


class DeviceOps:
    """Gradient sum and SGD step on the GPU: torch.distributed (NCCL) over a zero-copy view, cct_sgd_step."""

    def __init__(self, ctx, group=None):
        self.ctx, self.group = ctx, group

    def world_size(self):
        import torch.distributed as dist
        return dist.get_world_size(self.group) if dist.is_available() and dist.is_initialized() else 1

    def alloc(self, count):
        return self.ctx.malloc(4 * count)

    def view(self, ptr, count):
        import torch

        class _Iface:  # zero-copy: torch wraps the pointer through the CUDA array interface
            __cuda_array_interface__ = {"shape": (count,), "typestr": "<f4", "data": (ptr, False), "version": 3}

        return torch.as_tensor(_Iface(), device="cuda:%d" % self.ctx.device)

    def allreduce_sum(self, ptr, count):
        if self.world_size() > 1:
            import torch.distributed as dist
            dist.all_reduce(self.view(ptr, count), group=self.group)

    def sgd_step(self, count, w, g, h, lr, momentum, lam):
        vp = C.c_void_p
        capi.check(self.ctx.lib.cct_sgd_step(self.ctx.h, count, vp(w), vp(g), vp(h), lr, momentum, lam), "cct_sgd_step",
                   self.ctx.h)

    def zero(self, ptr, count):
        self.ctx.fill(ptr, count, 0.0)


class ParallelizedBridge:
    """One rank's share of a data-parallel convolution layer.

    `bridge` is this rank's sub-bridge over its batch slice (a ConvolutionBridge).  Its model, bias and gradient cubes
    are re-pointed into one flat buffer owned here, as the reference's ParallelizedBridge owns p_model_cube and hands
    the pointer to its sub-bridges (ParallelizedBridge_impl.hxx:519-532).
    """

    def __init__(self, bridge, solver, ops, lr_mult=(1.0, 2.0), decay_mult=(1.0, 0.0)):
        self.bridge, self.solver, self.ops = bridge, solver, ops
        self.n_w = bridge.p_model_cube.n_elements
        self.n_b = bridge.p_bias_cube.n_elements if bridge.bias_term else 0
        n = self.n_w + self.n_b
        self.count = n
        self.params, self.grads, self.hist = ops.alloc(n), ops.alloc(n), ops.alloc(n)
        ops.zero(self.hist, n)
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

    def backward(self):
        self.bridge.backward()
        self.ops.allreduce_sum(self.grads, self.count)  # gradients are summed, not averaged (:916-955)
        if not self.update_model_gradients:
            return
        s = self.solver
        self.current_iter += 1  # the updater increments before use (GradientUpdater.h:155)
        base = get_learning_rate(s.lr_policy, s.base_lr, s.gamma, float(self.current_iter), float(s.stepsize), s.power,
                                 float(s.max_iter))
        self.ops.sgd_step(self.n_w, self.params, self.grads, self.hist, float(np.float32(base * self.lr_mult[0])),
                          s.momentum, float(np.float32(s.weight_decay * self.decay_mult[0])))
        if self.n_b:
            off = 4 * self.n_w
            self.ops.sgd_step(self.n_b, self.params + off, self.grads + off, self.hist + off,
                              float(np.float32(base * self.lr_mult[1])), s.momentum,
                              float(np.float32(s.weight_decay * self.decay_mult[1])))
