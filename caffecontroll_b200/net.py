"""Prototxt-driven network construction and the training iteration, the slice of the reference's DeepNet that the hot
path needs (src/DeepNet.h:968-2030 construct_network, :171-266 run_forward_pass / run_backward_pass, :268-422 model
files), without protobuf or LMDB: a small reader for protobuf text format, a builder that turns the layer list into
bridges on one GPU (one batch partition per process), and the fusion pass that folds the parameter-free bridges into
the contractions around them.

Layer types handled: Data (shape only: inputs are fed by the caller), Convolution, ReLU, Pooling (MAX), LRN,
InnerProduct, Dropout, SoftmaxWithLoss - the types of the LeNet / CaffeNet / AlexNet prototxts of the reference's tests.
"""
import ctypes as C
import re

import numpy as np

from . import capi
from .bridge import ConvolutionBridge, FullyConnectedBridge, Layer, LogicalCube
from .layers import DropoutBridge, LRNBridge, MaxPoolingBridge, ReLUBridge, SoftmaxLossBridge
from .parallel import (DeviceOps, ModelParallelFullyConnectedBridge, ModelParallelizedBridge, ParallelizedBridge,
                       SolverParameter, model_parallel_gpus)

# ------------------------------------------------------------------------------------- protobuf text format

_TOKEN = re.compile(r'\s*(?:(#[^\n]*)|("(?:[^"\\]|\\.)*"|\'(?:[^\'\\]|\\.)*\')|([{}:<>\[\],;])|([^\s{}:<>\[\],;#"\']+))')


class Message(dict):
    """One parsed message: field name -> list of values (scalars or Messages), in file order."""

    def get1(self, name, default=None):
        v = self.get(name)
        return v[-1] if v else default

    def all(self, name):
        return self.get(name, [])

    def msg(self, name):
        v = self.get(name)
        return v[-1] if v else Message()


def _scalar(tok):
    if tok[0] in "\"'":
        return bytes(tok[1:-1], "utf-8").decode("unicode_escape")
    low = tok.lower()
    if low == "true":
        return True
    if low == "false":
        return False
    try:
        return int(tok, 0)
    except ValueError:
        pass
    try:
        return float(tok[:-1] if low.endswith("f") else tok)
    except ValueError:
        return tok  # an enum identifier


def parse_prototxt(text):
    """Parses protobuf text format (fields `name: value`, nested `name { ... }`, comments) into a Message."""
    toks, pos = [], 0
    while pos < len(text):
        m = _TOKEN.match(text, pos)
        if not m:
            if text[pos:].strip() == "":
                break
            raise ValueError("prototxt: cannot tokenise at offset %d: %r" % (pos, text[pos:pos + 20]))
        pos = m.end()
        if m.group(1) is None:
            toks.append(m.group(2) or m.group(3) or m.group(4))
    i = 0

    def message(closer):
        nonlocal i
        out = Message()
        while i < len(toks):
            t = toks[i]
            if t in ("}", ">"):
                if closer is None:
                    raise ValueError("prototxt: unbalanced %r" % t)
                i += 1
                return out
            if t in (",", ";"):
                i += 1
                continue
            name = t
            i += 1
            if i < len(toks) and toks[i] == ":":
                i += 1
            if i >= len(toks):
                raise ValueError("prototxt: field %r has no value" % name)
            if toks[i] in ("{", "<"):
                i += 1
                out.setdefault(name, []).append(message("}"))
            elif toks[i] == "[":
                i += 1
                while toks[i] != "]":
                    if toks[i] != ",":
                        out.setdefault(name, []).append(_scalar(toks[i]))
                    i += 1
                i += 1
            else:
                out.setdefault(name, []).append(_scalar(toks[i]))
                i += 1
        if closer is not None:
            raise ValueError("prototxt: missing closing brace")
        return out

    return message(None)


def solver_from_message(m):
    """cnn::SolverParameter fields the updater reads, with the schema's defaults (src/parser/cnn.proto)."""
    s = SolverParameter(base_lr=float(m.get1("base_lr", 0.01)), lr_policy=m.get1("lr_policy", "fixed"),
                        gamma=float(m.get1("gamma", 0.0)), stepsize=int(m.get1("stepsize", 1)),
                        power=float(m.get1("power", 0.0)), max_iter=int(m.get1("max_iter", 1)),
                        momentum=float(m.get1("momentum", 0.0)), weight_decay=float(m.get1("weight_decay", 0.0)),
                        regularization_type=m.get1("regularization_type", "L2"))
    s.random_seed = int(m.get1("random_seed", -1))
    return s


_TYPES = {"DATA": "Data", "CONVOLUTION": "Convolution", "RELU": "ReLU", "POOLING": "Pooling", "LRN": "LRN",
          "INNERPRODUCT": "InnerProduct", "INNER_PRODUCT": "InnerProduct", "DROPOUT": "Dropout",
          "SOFTMAXWITHLOSS": "SoftmaxWithLoss", "SOFTMAX_LOSS": "SoftmaxWithLoss", "ACCURACY": "Accuracy"}


def _layer_type(layer):
    t = str(layer.get1("type", ""))
    return _TYPES.get(t.upper(), t)


def _in_phase(layer, phase):
    for inc in layer.all("include"):
        p = inc.get1("phase")
        if p is not None and str(p).upper() != phase:
            return False
    return True


def _multipliers(layer):
    """(lr_mult, decay_mult) for (weights, bias): `param { lr_mult decay_mult }` blocks, or the older per-blob
    `blobs_lr` / `weight_decay` lists (src/bridges/ParallelizedBridge_impl.hxx:39-75); default 1, 1."""
    lr, decay = [1.0, 1.0], [1.0, 1.0]
    params = layer.all("param")
    if params and isinstance(params[0], Message):
        for j, p in enumerate(params[:2]):
            lr[j], decay[j] = float(p.get1("lr_mult", 1.0)), float(p.get1("decay_mult", 1.0))
    else:
        for j, v in enumerate(layer.all("blobs_lr")[:2]):
            lr[j] = float(v)
        for j, v in enumerate(layer.all("weight_decay")[:2]):
            decay[j] = float(v)
    return tuple(lr), tuple(decay)


def _fill(ctx, cube, filler, random_seed, n_batch):
    """ConvolutionBridge::initialize_logical_cube (src/bridges/ConvolutionBridge_impl.hxx:250-267)."""
    kind = str(filler.get1("type", "constant"))
    lib, vp = ctx.lib, C.c_void_p
    if kind == "constant":
        ctx.fill(cube.ptr, cube.n_elements, float(filler.get1("value", 0.0)))
        return
    table = {"gaussian": (capi.FILL_GAUSSIAN, float(filler.get1("mean", 0.0)), float(filler.get1("std", 1.0))),
             "xavier": (capi.FILL_XAVIER, float(cube.n_elements // n_batch), 0.0),
             "bernoulli": (capi.FILL_BERNOULLI, float(filler.get1("value", 0.0)), 0.0)}
    if kind not in table:
        raise ValueError("filler type %r is not supported" % kind)
    k, a, b = table[kind]
    capi.check(lib.cct_fill_random(ctx.h, vp(cube.ptr), cube.n_elements, k, a, b, random_seed), "cct_fill_random", ctx.h)


class Net:
    """The bridges of one network on one GPU, in execution order, plus the per-layer updaters.

    forward() / backward() run the bridge list as DeepNet::run_forward_pass / run_backward_pass do; backward() hands
    each parameterised layer's gradients to the all-reduce as soon as the layer's backward pass is queued (so the
    reduction overlaps the layers below), and applies the SGD updates once all of them have been reduced.
    """

    def __init__(self, ctx, net_param, solver, batch, input_shape=None, ops=None, fuse=True, loss_batch=None,
                 algo=capi.ALGO_AUTO, phase="TRAIN", model_parallel=()):
        """model_parallel: names of InnerProduct layers to split over all ranks by output depth, beside those whose
        placement fields (gpu_N_depth_proportion) ask for it - the fields only reach four GPUs."""
        self.ctx, self.solver, self.batch = ctx, solver, batch
        self.ops = ops or DeviceOps(ctx)
        self.blobs, self.bridges, self.names, self.types = {}, [], [], []
        self.pbridges = {}          # index in self.bridges -> ParallelizedBridge (layers with parameters)
        self.labels = None
        self.loss_bridge = None
        self.flops_forward = 0.0    # multiply-adds x 2 of the forward contractions (each counted once)
        self.flops_backward = 0.0
        self._cubes = []
        seed = getattr(solver, "random_seed", -1)
        layers = [l for l in net_param.all("layer") + net_param.all("layers") if _in_phase(l, phase)]
        first_param_layer = True
        for layer in layers:
            typ, name = _layer_type(layer), str(layer.get1("name", ""))
            bottoms, tops = [str(b) for b in layer.all("bottom")], [str(t) for t in layer.all("top")]
            if typ == "Data":
                if input_shape is None:
                    crop = layer.msg("transform_param").get1("crop_size") or layer.msg("data_param").get1("crop_size")
                    if not crop:
                        raise ValueError("data layer %r: give input_shape=(channels, size)" % name)
                    input_shape = (3, int(crop))
                D, n = input_shape
                self.blobs[tops[0]] = self._layer(n, n, D, with_grad=False)
                if len(tops) > 1:
                    self.labels = LogicalCube(ctx, 1, 1, 1, batch)
                    self._cubes.append(self.labels)
                continue
            if typ == "Accuracy":
                continue  # a test-phase metric, not part of the training iteration
            src = self.blobs[bottoms[0]]
            x = src.p_data_cube
            if typ == "Convolution":
                cp = layer.msg("convolution_param")
                k, s, p = int(cp.get1("kernel_size")), int(cp.get1("stride", 1)), int(cp.get1("pad", 0))
                o, g = int(cp.get1("num_output")), int(cp.get1("group", 1))
                m = (x.R + 2 * p - k) // s + 1
                dst = self._top(tops[0], bottoms[0], m, m, o)
                br = ConvolutionBridge(src, dst, k, s, p, g, bool(cp.get1("bias_term", True)), algo, ctx)
                _fill(ctx, br.p_model_cube, cp.msg("weight_filler"), seed, o)
                if br.bias_term:
                    _fill(ctx, br.p_bias_cube, cp.msg("bias_filler"), seed, 1)
                F = 2.0 * o * (k * k * x.D // g) * m * m * batch
            elif typ == "InnerProduct":
                ip = layer.msg("inner_product_param")
                o = int(ip.get1("num_output"))
                dst = self._top(tops[0], bottoms[0], 1, 1, o)
                comm = getattr(self.ops, "comm", None)
                shares = [float(layer.get1("gpu_%d_depth_proportion" % g, 0.0)) for g in range(4)]
                gpus = model_parallel_gpus(shares, o)  # src/DeepNet.h:728-790
                if gpus and (comm is None or comm.nranks != len(gpus)):
                    raise ValueError("layer %r asks for model parallelism over %d GPUs; the job has %d rank(s)" %
                                     (name, len(gpus), comm.nranks if comm is not None else 1))
                if name in model_parallel and (comm is None or comm.nranks < 2):
                    raise ValueError("layer %r: model parallelism needs a communicator of two or more ranks" % name)
                if gpus or name in model_parallel:
                    # src/DeepNet.h:1213-1357.  The slices are cut from the matrix the fillers give the whole layer, so
                    # the net starts from the same parameters as its data-parallel form with the same seed (the
                    # reference fills every slice bridge from the same seed, which makes the slices copies of each other).
                    br = ModelParallelFullyConnectedBridge(src, dst, comm, bool(ip.get1("bias_term", True)), algo, ctx)
                    whole = LogicalCube(ctx, x.R, x.C, x.D, o)
                    _fill(ctx, whole, ip.msg("weight_filler"), seed, o)
                    n = br.p_model_cube.n_elements
                    self.ops.copy(br.p_model_cube.ptr, whole.ptr + 4 * comm.rank * n, n)
                    whole.free()
                    if br.bias_term:
                        whole = LogicalCube(ctx, 1, 1, o, 1)
                        _fill(ctx, whole, ip.msg("bias_filler"), seed, 1)
                        self.ops.copy(br.p_bias_cube.ptr, whole.ptr + 4 * comm.rank * br.slice_depth, br.slice_depth)
                        whole.free()
                else:
                    br = FullyConnectedBridge(src, dst, bool(ip.get1("bias_term", True)), algo, ctx)
                    _fill(ctx, br.p_model_cube, ip.msg("weight_filler"), seed, o)
                    if br.bias_term:
                        _fill(ctx, br.p_bias_cube, ip.msg("bias_filler"), seed, 1)
                F = 2.0 * o * (x.R * x.C * x.D) * batch
            elif typ == "ReLU":
                br = ReLUBridge(src, self._top(tops[0], bottoms[0], x.R, x.C, x.D), ctx)
            elif typ == "Pooling":
                pp = layer.msg("pooling_param")
                if str(pp.get1("pool", "MAX")).upper() not in ("MAX", "0"):
                    raise ValueError("layer %r: only MAX pooling is built" % name)
                k, s = int(pp.get1("kernel_size")), int(pp.get1("stride", 1))
                m = (x.R - k) // s + 1  # floor, as src/DeepNet.h:112-115 computes it
                br = MaxPoolingBridge(src, self._top(tops[0], bottoms[0], m, m, x.D), k, s, ctx)
            elif typ == "LRN":
                lp = layer.msg("lrn_param")
                br = LRNBridge(src, self._top(tops[0], bottoms[0], x.R, x.C, x.D), int(lp.get1("local_size", 5)),
                               float(lp.get1("alpha", 1.0)), float(lp.get1("beta", 0.75)), ctx)
            elif typ == "Dropout":
                ratio = float(layer.msg("dropout_param").get1("dropout_ratio", 0.5))
                br = DropoutBridge(src, self._top(tops[0], bottoms[0], x.R, x.C, x.D), ratio, seed, ctx)
            elif typ == "SoftmaxWithLoss":
                if self.labels is None:
                    self.labels = LogicalCube(ctx, 1, 1, 1, batch)
                    self._cubes.append(self.labels)
                br = SoftmaxLossBridge(src, self._top(tops[0] if tops else name, None, x.R, x.C, x.D), self.labels,
                                       loss_batch or batch, ctx)
                self.loss_bridge = br
            else:
                raise ValueError("layer %r: type %r is not built" % (name, typ))
            if typ in ("Convolution", "InnerProduct"):
                if first_param_layer:
                    br.needs_to_calc_backward_grad = False  # nothing below the first layer wants dX (src/DeepNet.h:1108-1110)
                    first_param_layer = False
                lr_mult, decay_mult = _multipliers(layer)
                if isinstance(br, ModelParallelFullyConnectedBridge):
                    pb = ModelParallelizedBridge(br, solver, ctx, lr_mult, decay_mult, defer_update=True)
                else:
                    pb = ParallelizedBridge(br, solver, self.ops, lr_mult, decay_mult, defer_update=True)
                self.pbridges[len(self.bridges)] = pb
                self.flops_forward += F
                self.flops_backward += (2.0 if br.needs_to_calc_backward_grad else 1.0) * F
            self.bridges.append(br)
            self.names.append(name)
            self.types.append(typ)
        self.in_place = [self.bridges[i].p_input_layer is self.bridges[i].p_output_layer for i in range(len(self.bridges))]
        self.input = next(iter(self.blobs.values()))
        self.fused = []
        if fuse:
            self._fuse()

    # ---- construction helpers
    def _layer(self, R, Cc, D, with_grad=True):
        data = LogicalCube(self.ctx, R, Cc, D, self.batch)
        grad = LogicalCube(self.ctx, R, Cc, D, self.batch) if with_grad else None
        self._cubes += [c for c in (data, grad) if c is not None]
        return Layer(data, grad)

    def _top(self, top, bottom, R, Cc, D):
        if top == bottom:  # in place: the bridge reads and writes the same layer
            return self.blobs[bottom]
        self.blobs[top] = self._layer(R, Cc, D)
        return self.blobs[top]

    # ---- fusion: fold the parameter-free bridges into the contractions around them
    def _fuse(self):
        B, T = self.bridges, self.types

        def consumer_of(i):  # the next bridge that reads bridge i's output layer, if it is the very next one
            j = i + 1
            return j if j < len(B) and B[j].p_input_layer is B[i].p_output_layer else None

        def tensor_core(br):
            return br.algo == capi.ALGO_UMMA_3XTF32 and (not isinstance(br, FullyConnectedBridge) or br.plan)

        for i, br in enumerate(B):
            if T[i] not in ("Convolution", "InnerProduct") or not tensor_core(br):
                continue
            r = consumer_of(i)
            if r is None or T[r] != "ReLU" or not self.in_place[r]:
                continue
            nxt = consumer_of(r)
            if nxt is None:
                continue
            if T[i] == "Convolution" and T[nxt] == "Pooling":
                pool = B[nxt]
                br.fuse_relu = True
                # the pooled tensor gives the ReLU mask unless a later in-place layer overwrites it before backward
                after = nxt + 1
                pooled_intact = not (after < len(B) and self.in_place[after] and B[after].p_input_layer is pool.p_output_layer)
                br.fuse_pool_relu_backward(pool.p_output_layer.p_gradient_cube, pool.max_index, pool.kernel_size, pool.stride,
                                           pool.p_output_layer.p_data_cube if pooled_intact else None)
                B[r].skip_forward = B[r].skip_backward = pool.skip_backward = True
                self.fused.append("%s+%s(+%s backward)" % (self.names[i], self.names[r], self.names[nxt]))
            elif T[nxt] in ("Convolution", "InnerProduct") and tensor_core(B[nxt]):
                br.fuse_relu = True
                B[nxt].fuse_relu_backward = True
                B[r].skip_forward = B[r].skip_backward = True
                self.fused.append("%s+%s, mask in %s" % (self.names[i], self.names[r], self.names[nxt]))
            elif (T[i] == "InnerProduct" and T[nxt] == "Dropout" and self.in_place[nxt] and consumer_of(nxt) is not None and
                  T[consumer_of(nxt)] == "InnerProduct" and tensor_core(B[consumer_of(nxt)])):
                drop, cons = B[nxt], B[consumer_of(nxt)]
                br.fuse_relu = True
                br.dropout_mask, br.dropout_scale = drop.mask_cube, drop.scale
                cons.fuse_relu_backward = True
                cons.input_dropout_mask, cons.input_dropout_scale = drop.mask_cube, drop.scale
                B[r].skip_forward = B[r].skip_backward = True
                drop.skip_forward = drop.skip_backward = True
                # the mask must exist before the layer that applies it runs: draw it in the producer's slot
                self.bridges[i] = _WithPrologue(br, drop.draw_mask)
                drop.draw_mask = lambda: None
                self.fused.append("%s+%s+%s, masks in %s" % (self.names[i], self.names[r], self.names[nxt],
                                                             self.names[consumer_of(nxt)]))

    # ---- data in, results out
    def set_input(self, X, labels=None):
        self.input.p_data_cube.upload(X)
        if labels is not None and self.labels is not None:
            self.labels.upload(np.ascontiguousarray(labels, dtype=np.float32).reshape(self.labels.shape))

    def blob(self, name, grad=False):
        layer = self.blobs[name]
        return (layer.p_gradient_cube if grad else layer.p_data_cube).download()

    def get_loss(self):
        return self.loss_bridge.get_loss() if self.loss_bridge else None

    def read_loss_into(self, host_ptr):
        """Asynchronous form of get_loss(): see SoftmaxLossBridge.read_loss_into."""
        self.loss_bridge.read_loss_into(host_ptr)

    def param_bridges(self):
        return [(self.names[i], self.pbridges[i]) for i in sorted(self.pbridges)]

    # ---- the iteration
    def forward(self):
        for i, br in enumerate(self.bridges):
            br.forward()

    def backward(self):
        # Gradient sums are begun per layer and run on the communicator's stream beside the layers below.  The fully
        # connected layers' sums (most of the bytes) are held back until the first convolution's backward pass is next:
        # the inner-product kernels are single-wave grids that lose a whole wave when NCCL takes SMs away from them,
        # the convolution kernels are many-round persistent grids that only slow down in proportion.
        held = []
        for i in range(len(self.bridges) - 1, -1, -1):
            pb = self.pbridges.get(i)
            if pb is not None:
                if self.types[i] == "InnerProduct":
                    pb.backward(begin_allreduce=False)
                    held.append(pb)
                else:
                    for h in held:
                        h.begin_allreduce()
                    held = []
                    pb.backward()   # sub-bridge backward, then the gradient all-reduce is begun (not waited for)
            else:
                self.bridges[i].backward()
        for h in held:
            h.begin_allreduce()
        self.ops.allreduce_wait()
        for i in sorted(self.pbridges, reverse=True):
            self.pbridges[i].apply_update()

    def step(self):
        self.forward()
        self.backward()

    def set_update_model_gradients(self, flag):
        for pb in self.pbridges.values():
            pb.set_update_model_gradients(flag)

    # ---- model files (src/DeepNet.h:331-376): raw fp32, bridges in execution order, model then bias
    def write_model_to_file(self, path):
        self.ctx.sync()
        with open(path, "wb") as f:
            for _, pb in self.param_bridges():
                if hasattr(pb, "model_host"):  # a layer split over the ranks: the whole matrix, gathered (a collective)
                    w, b = pb.model_host()
                    w.astype(np.float32).tofile(f)
                    if b is not None:
                        b.astype(np.float32).tofile(f)
                    continue
                pb.get_model_cube().download().astype(np.float32).tofile(f)
                if pb.get_bias_cube() is not None:
                    pb.get_bias_cube().download().astype(np.float32).tofile(f)

    def read_model_from_file(self, path):
        with open(path, "rb") as f:
            for name, pb in self.param_bridges():
                if hasattr(pb, "set_model_host"):  # a layer split over the ranks keeps its own rows
                    n_w, n_b = pb.full_counts
                    w, b = np.fromfile(f, np.float32, n_w), (np.fromfile(f, np.float32, n_b) if n_b else None)
                    if w.size != n_w or (b is not None and b.size != n_b):
                        raise ValueError("model file ends inside layer %r" % name)
                    pb.set_model_host(w, b)
                    continue
                for cube in (pb.get_model_cube(), pb.get_bias_cube()):
                    if cube is None:
                        continue
                    a = np.fromfile(f, np.float32, cube.n_elements)
                    if a.size != cube.n_elements:
                        raise ValueError("model file ends inside layer %r" % name)
                    cube.upload(a.reshape(cube.shape))
            if f.read(1):
                raise ValueError("model file is longer than the network's parameters")

    # ---- snapshots (src/DeepNet.h:268-328): the model file, the momentum history in the same order, and the iteration
    def write_snapshot(self, prefix):
        """Writes <prefix>.MODEL, <prefix>.HISTORY and <prefix>.ITER."""
        self.write_model_to_file(prefix + ".MODEL")
        with open(prefix + ".HISTORY", "wb") as f:
            for _, pb in self.param_bridges():
                w, b = pb.history_host()
                w.tofile(f)
                if b is not None:
                    b.tofile(f)
        it = max([pb.current_iter for pb in self.pbridges.values()] or [0])
        with open(prefix + ".ITER", "w") as f:
            f.write("%d\n" % it)

    def read_snapshot(self, prefix):
        self.read_model_from_file(prefix + ".MODEL")
        with open(prefix + ".HISTORY", "rb") as f:
            for name, pb in self.param_bridges():
                n_w, n_b = getattr(pb, "full_counts", (pb.n_w, pb.n_b))
                w = np.fromfile(f, np.float32, n_w)
                b = np.fromfile(f, np.float32, n_b) if n_b else None
                if w.size != n_w or (b is not None and b.size != n_b):
                    raise ValueError("history file ends inside layer %r" % name)
                pb.set_history_host(w, b)
        with open(prefix + ".ITER") as f:
            it = int(f.read().split()[0])
        for pb in self.pbridges.values():
            pb.set_current_iter(it)

    def num_parameters(self):
        return sum(pb.count for pb in self.pbridges.values())

    def launches_per_step(self):
        """Kernels one forward + backward + update launches, counted from the structure of the calls: convolution
        forward = weight pack + contraction; its backward = weight gradient (dY split + contraction + split reduction +
        bias sums for lowered matrices of 512 rows or more, else contraction + reduction), data gradient (pack +
        contraction), plus one pass per folded mask; fully connected = contraction + reduction per pass, bias sums;
        one kernel per parameter-free bridge pass; two SGD kernels per parameterised layer."""
        n = 0
        for i, br in enumerate(self.bridges):
            t = self.types[i]
            if t == "Convolution":
                wg = 4 if (br.iD // br.group) * br.K * br.K >= 512 else 2
                n += 2 + wg + (2 if br.needs_to_calc_backward_grad else 0)
                n += (1 if br.pool_fusion is not None else 0) + (1 if br.fuse_relu_backward and br.needs_to_calc_backward_grad else 0)
            elif t == "InnerProduct":
                n += 2 + 2 + (2 if br.needs_to_calc_backward_grad else 0)
            elif t == "SoftmaxWithLoss":
                n += 3
            elif t == "Dropout":
                n += 1 + (0 if br.skip_forward else 1) + (0 if br.skip_backward else 1)
            elif t == "Pooling":
                n += 1 + (0 if br.skip_backward else 1)
            else:
                n += (0 if br.skip_forward else 1) + (0 if br.skip_backward else 1)
        return n + 2 * len(self.pbridges)

    def close(self):
        self.ctx.sync()
        for br in self.bridges:
            br.close()
        for pb in self.pbridges.values():
            pb.close()
        for c in self._cubes:
            c.free()
        self._cubes = []


class _WithPrologue:
    """A bridge whose forward() is preceded by a host-side action (drawing the dropout mask it applies)."""

    def __init__(self, bridge, prologue):
        object.__setattr__(self, "_bridge", bridge)
        object.__setattr__(self, "_prologue", prologue)

    def forward(self):
        self._prologue()
        self._bridge.forward()

    def __getattr__(self, name):
        return getattr(self._bridge, name)

    def __setattr__(self, name, value):
        setattr(self._bridge, name, value)


def load_net(ctx, net_text, solver_text, batch, **kw):
    """Builds a Net from the text of a net prototxt and a solver prototxt."""
    return Net(ctx, parse_prototxt(net_text), solver_from_message(parse_prototxt(solver_text)), batch, **kw)
