"""Host-side mirrors of the reference's parameter-free bridges, on top of the C ABI: ReLUBridge, MaxPoolingBridge,
LRNBridge, DropoutBridge, SoftmaxLossBridge (src/bridges/*Bridge.h).  Same constructor shape everywhere - an input Layer
and an output Layer - and the same forward() / backward() pair as PhysicalOperator (src/bridges/PhysicalOperator.h:15-30).
A network may mark a bridge's pass as folded into a neighbouring contraction (skip_forward / skip_backward); the bridge
then does nothing in that pass.
"""
import ctypes as C

import numpy as np

from . import capi
from .bridge import LogicalCube

_vp = C.c_void_p


class _Bridge:
    def __init__(self, p_input_layer, p_output_layer, ctx=None):
        self.p_input_layer, self.p_output_layer = p_input_layer, p_output_layer
        x, y = p_input_layer.p_data_cube, p_output_layer.p_data_cube
        self.ctx = ctx or x.ctx
        self.lib = self.ctx.lib
        self.iR, self.iC, self.iD, self.iB = x.R, x.C, x.D, x.B
        self.oR, self.oC, self.oD, self.oB = y.R, y.C, y.D, y.B
        self.needs_to_calc_backward_grad = True
        self.skip_forward = False   # folded into the producing contraction's epilogue
        self.skip_backward = False  # folded into a neighbouring contraction's backward pass

    def close(self):
        pass


class ReLUBridge(_Bridge):
    """src/bridges/ReLUBridge_impl.hxx:36-99: Y = max(X, 0); dX = dY * [X > 0].  Input and output may be the same
    layer (in place), in which case the mask is read from the output (Y > 0 exactly where X > 0)."""

    def forward(self):
        if self.skip_forward:
            return
        x, y = self.p_input_layer.p_data_cube, self.p_output_layer.p_data_cube
        capi.check(self.lib.cct_relu_forward(self.ctx.h, _vp(x.ptr), _vp(y.ptr), x.n_elements), "cct_relu_forward", self.ctx.h)

    def backward(self):
        if self.skip_backward or not self.needs_to_calc_backward_grad:
            return
        y = self.p_output_layer.p_data_cube
        dy, dx = self.p_output_layer.p_gradient_cube, self.p_input_layer.p_gradient_cube
        capi.check(self.lib.cct_relu_backward(self.ctx.h, _vp(y.ptr), _vp(dy.ptr), _vp(dx.ptr), y.n_elements),
                   "cct_relu_backward", self.ctx.h)


class MaxPoolingBridge(_Bridge):
    """src/bridges/MaxPoolingBridge_impl.hxx:36-151: k x k windows with stride s, no padding, output size by floor;
    the arg-max offsets of the forward pass (max_index) route the gradient."""

    def __init__(self, p_input_layer, p_output_layer, kernel_size, stride, ctx=None):
        super().__init__(p_input_layer, p_output_layer, ctx)
        self.kernel_size, self.stride = kernel_size, stride
        m = (self.iR - kernel_size) // stride + 1
        if (self.oR, self.oC, self.oD, self.oB) != (m, m, self.iD, self.iB) or self.iR != self.iC:
            raise ValueError("pooling output layer must be %dx%dxD%dxB%d" % (m, m, self.iD, self.iB))
        self.max_index = LogicalCube(self.ctx, m, m, self.iD, self.iB, np.int32)

    def forward(self):
        x, y = self.p_input_layer.p_data_cube, self.p_output_layer.p_data_cube
        capi.check(self.lib.cct_maxpool_forward(self.ctx.h, _vp(x.ptr), _vp(y.ptr), _vp(self.max_index.ptr),
                                                self.iB * self.iD, self.iR, self.kernel_size, self.stride),
                   "cct_maxpool_forward", self.ctx.h)

    def backward(self):
        if self.skip_backward or not self.needs_to_calc_backward_grad:
            return
        dy, dx = self.p_output_layer.p_gradient_cube, self.p_input_layer.p_gradient_cube
        capi.check(self.lib.cct_maxpool_backward(self.ctx.h, _vp(dy.ptr), _vp(self.max_index.ptr), _vp(dx.ptr),
                                                 self.iB * self.iD, self.iR, self.kernel_size, self.stride),
                   "cct_maxpool_backward", self.ctx.h)

    def close(self):
        self.max_index.free()


class LRNBridge(_Bridge):
    """src/bridges/LRNBridge_impl.hxx:46-190 (across channels).  The reference's bridge keeps a cube of denominators
    (`denoms`) from its forward pass for its backward pass; here that cube is optional (keep_denoms): for windows of 3 and
    5 channels the backward kernel forms the denominators again from the input, which costs less than writing and
    reading them (8 B per element of HBM traffic in each pass).  Other windows always keep it."""

    def __init__(self, p_input_layer, p_output_layer, local_size=5, alpha=1.0, beta=0.75, ctx=None, keep_denoms=False):
        super().__init__(p_input_layer, p_output_layer, ctx)
        if local_size % 2 != 1:
            raise ValueError("local_size must be odd")
        self.local_size, self.alpha, self.beta = local_size, alpha, beta
        keep = keep_denoms or local_size not in (3, 5)
        self.denoms = LogicalCube(self.ctx, self.iR, self.iC, self.iD, self.iB) if keep else None

    def forward(self):
        x, y = self.p_input_layer.p_data_cube, self.p_output_layer.p_data_cube
        capi.check(self.lib.cct_lrn_forward(self.ctx.h, _vp(x.ptr), _vp(y.ptr), _vp(self.denoms.ptr if self.denoms else None),
                                            self.iB, self.iD, self.iR * self.iC, self.local_size, self.alpha, self.beta),
                   "cct_lrn_forward", self.ctx.h)

    def backward(self):
        if not self.needs_to_calc_backward_grad:
            return
        x, y = self.p_input_layer.p_data_cube, self.p_output_layer.p_data_cube
        dy, dx = self.p_output_layer.p_gradient_cube, self.p_input_layer.p_gradient_cube
        capi.check(self.lib.cct_lrn_backward(self.ctx.h, _vp(x.ptr), _vp(y.ptr), _vp(self.denoms.ptr if self.denoms else None),
                                             _vp(dy.ptr), _vp(dx.ptr), self.iB, self.iD, self.iR * self.iC, self.local_size,
                                             self.alpha, self.beta), "cct_lrn_backward", self.ctx.h)

    def close(self):
        if self.denoms is not None:
            self.denoms.free()


class DropoutBridge(_Bridge):
    """src/bridges/DropoutBridge_impl.hxx:49-175 in the training phase: a fresh mask per forward pass, output =
    input * mask * 1 / (1 - ratio), the same product on the gradient.  The mask is drawn on the device from
    (random_seed, pass counter); set_mask() injects a given one (parity runs use the CPU oracle's)."""

    def __init__(self, p_input_layer, p_output_layer, dropout_ratio=0.5, random_seed=1, ctx=None):
        super().__init__(p_input_layer, p_output_layer, ctx)
        self.dropout_ratio = dropout_ratio
        self.scale = 1.0 / (1.0 - dropout_ratio)
        self.random_seed = random_seed if random_seed >= 0 else int(np.random.SeedSequence().entropy % (1 << 62))
        self.mask_cube = LogicalCube(self.ctx, self.iR, self.iC, self.iD, self.iB, np.uint32)
        self.calls = 0
        self.injected = False

    def set_mask(self, mask):
        self.mask_cube.upload(np.ascontiguousarray(mask, dtype=np.uint32))
        self.injected = True

    def draw_mask(self):
        if self.injected:
            return
        self.calls += 1
        capi.check(self.lib.cct_dropout_mask(self.ctx.h, _vp(self.mask_cube.ptr), self.mask_cube.n_elements,
                                             self.dropout_ratio, self.random_seed, self.calls), "cct_dropout_mask", self.ctx.h)

    def forward(self):
        self.draw_mask()
        if self.skip_forward:
            return
        x, y = self.p_input_layer.p_data_cube, self.p_output_layer.p_data_cube
        capi.check(self.lib.cct_dropout_apply(self.ctx.h, _vp(x.ptr), _vp(self.mask_cube.ptr), self.scale, _vp(y.ptr),
                                              x.n_elements), "cct_dropout_apply", self.ctx.h)

    def backward(self):
        if self.skip_backward or not self.needs_to_calc_backward_grad:
            return
        dy, dx = self.p_output_layer.p_gradient_cube, self.p_input_layer.p_gradient_cube
        capi.check(self.lib.cct_dropout_apply(self.ctx.h, _vp(dy.ptr), _vp(self.mask_cube.ptr), self.scale, _vp(dx.ptr),
                                              dy.n_elements), "cct_dropout_apply", self.ctx.h)

    def close(self):
        self.mask_cube.free()


class SoftmaxLossBridge(_Bridge):
    """src/bridges/SoftmaxLossBridge_impl.hxx:36-145 (host-only in the reference; a device kernel here): the output
    layer receives the probabilities, get_loss() the summed loss, backward() writes (prob - onehot) / loss_batch into
    the input layer's gradient.  loss_batch is the batch the loss is averaged over: this partition's batch in a
    single-GPU run, the whole job's in a data-parallel one (the reference sizes its label cube to the full batch,
    src/DeepNet.h:1909-1912), so that the partitions' gradients add up to the full-batch gradient."""

    def __init__(self, p_input_layer, p_output_layer, p_data_labels, loss_batch=None, ctx=None):
        super().__init__(p_input_layer, p_output_layer, ctx)
        self.p_data_labels = p_data_labels
        self.classes = self.iR * self.iC * self.iD
        self.loss_batch = loss_batch or self.iB
        self.image_loss = LogicalCube(self.ctx, 1, 1, 1, self.iB)
        self.loss_cube = LogicalCube(self.ctx, 1, 1, 1, 1)

    def forward(self):
        x, y = self.p_input_layer.p_data_cube, self.p_output_layer.p_data_cube
        capi.check(self.lib.cct_softmax_loss_forward(self.ctx.h, _vp(x.ptr), _vp(self.p_data_labels.ptr), _vp(y.ptr),
                                                     _vp(self.image_loss.ptr), _vp(self.loss_cube.ptr), self.iB,
                                                     self.classes), "cct_softmax_loss_forward", self.ctx.h)

    def backward(self):
        y, dx = self.p_output_layer.p_data_cube, self.p_input_layer.p_gradient_cube
        capi.check(self.lib.cct_softmax_loss_backward(self.ctx.h, _vp(y.ptr), _vp(self.p_data_labels.ptr), _vp(dx.ptr),
                                                      self.iB, self.classes, 1.0 / self.loss_batch),
                   "cct_softmax_loss_backward", self.ctx.h)

    def get_loss(self):
        """Summed loss of this partition's images (a device-to-host read: synchronises the stream)."""
        return float(self.loss_cube.download().reshape(-1)[0])

    def read_loss_into(self, host_ptr):
        """Queues the copy of the summed loss (one float) into pinned host memory at `host_ptr`, behind the kernels already
        on the stream, without waiting for it: a training loop reads the value once the stream has passed that point
        (an event, or the next synchronisation) and so never stalls the launches of the following iteration."""
        capi.check(self.lib.cct_memcpy_d2h(self.ctx.h, _vp(host_ptr), _vp(self.loss_cube.ptr), 4), "cct_memcpy_d2h", self.ctx.h)

    def close(self):
        self.image_loss.free()
        self.loss_cube.free()
