"""Host-side mirror of the reference's operator interface for the convolution path, on top of the C ABI.

Names follow the reference: LogicalCube (R x C x D x B, c fastest = NCHW; src/LogicalCube.h), Layer (a data cube
and a gradient cube; src/Layer.h:36-37), ConvolutionBridge with forward()/backward(), needs_to_calc_backward_grad,
bias_term, set_model_cube/get_model_cube/... (src/bridges/AbstractBridge.h:25-223, src/bridges/ConvolutionBridge.h).
Cubes live in device memory; numpy arrays cross the boundary only through upload()/download().
"""
import ctypes as C

import numpy as np

from . import capi


class Context:
    """One device context (stream + status word); replaces the reference's GPUDriver instance."""

    def __init__(self, device=0, stream=None):
        self.lib = capi.load()
        h = C.c_void_p()
        if stream is None:
            capi.check(self.lib.cct_ctx_create(device, C.byref(h)), "cct_ctx_create")
        else:
            capi.check(self.lib.cct_ctx_create_on_stream(device, C.c_void_p(stream), C.byref(h)),
                       "cct_ctx_create_on_stream")
        self.h = h
        self.device = device
        self.stream = stream  # the cudaStream_t the context enqueues on when the caller supplied one, else None

    def close(self):
        if self.h:
            self.lib.cct_ctx_destroy(self.h)
            self.h = None

    def sync(self):
        capi.check(self.lib.cct_sync(self.h), "cct_sync", self.h)

    def malloc(self, nbytes):
        p = C.c_void_p()
        capi.check(self.lib.cct_malloc(self.h, nbytes, C.byref(p)), "cct_malloc", self.h)
        return p.value

    def free(self, ptr):
        capi.check(self.lib.cct_free(self.h, C.c_void_p(ptr)), "cct_free", self.h)

    def h2d(self, ptr, arr):
        arr = np.ascontiguousarray(arr)
        capi.check(self.lib.cct_memcpy_h2d(self.h, C.c_void_p(ptr), arr.ctypes.data_as(C.c_void_p), arr.nbytes),
                   "cct_memcpy_h2d", self.h)
        self.sync()  # the numpy source may be a temporary

    def d2h(self, arr, ptr):
        assert arr.flags["C_CONTIGUOUS"]
        capi.check(self.lib.cct_memcpy_d2h(self.h, arr.ctypes.data_as(C.c_void_p), C.c_void_p(ptr), arr.nbytes),
                   "cct_memcpy_d2h", self.h)
        self.sync()

    def fill(self, ptr, count, value):
        capi.check(self.lib.cct_fill_f32(self.h, C.c_void_p(ptr), count, value), "cct_fill_f32", self.h)


class LogicalCube:
    """R x C x D x B fp32 (or int32) cube in device memory; numpy view of it is shaped (B, D, R, C)."""

    def __init__(self, ctx, R, C_, D, B, dtype=np.float32, ptr=None):
        self.ctx, self.R, self.C, self.D, self.B = ctx, R, C_, D, B
        self.dtype = np.dtype(dtype)
        self.n_elements = R * C_ * D * B
        self.own_data = ptr is None
        self.ptr = ctx.malloc(self.n_elements * self.dtype.itemsize) if ptr is None else ptr

    @property
    def shape(self):
        return (self.B, self.D, self.R, self.C)

    @classmethod
    def from_numpy(cls, ctx, arr):
        arr = np.ascontiguousarray(arr)
        shape = (1,) * (4 - arr.ndim) + arr.shape
        B, D, R, Cc = shape
        cube = cls(ctx, R, Cc, D, B, arr.dtype)
        ctx.h2d(cube.ptr, arr)
        return cube

    def upload(self, arr):
        arr = np.ascontiguousarray(arr, dtype=self.dtype)
        assert arr.size == self.n_elements
        self.ctx.h2d(self.ptr, arr)

    def download(self):
        out = np.empty(self.shape, self.dtype)
        self.ctx.d2h(out, self.ptr)
        return out

    def reset_cube(self, value=0.0):
        self.ctx.fill(self.ptr, self.n_elements, value)

    def free(self):
        if self.own_data and self.ptr:
            self.ctx.free(self.ptr)
            self.ptr = None


class Layer:
    def __init__(self, p_data_cube, p_gradient_cube):
        self.p_data_cube = p_data_cube
        self.p_gradient_cube = p_gradient_cube


class ConvolutionBridge:
    """forward(): p_input_layer.p_data_cube -> p_output_layer.p_data_cube.
    backward(): p_output_layer.p_gradient_cube (+ input data) -> p_input_layer.p_gradient_cube (iff
    needs_to_calc_backward_grad), model gradient and bias gradient cubes (overwritten)."""

    def __init__(self, p_input_layer, p_output_layer, kernel_size, stride=1, pad=0, group=1, bias_term=True,
                 algo=capi.ALGO_AUTO, ctx=None):
        self.p_input_layer, self.p_output_layer = p_input_layer, p_output_layer
        x, y = p_input_layer.p_data_cube, p_output_layer.p_data_cube
        self.ctx = ctx or x.ctx
        self.lib = self.ctx.lib
        self.iR, self.iC, self.iD, self.iB = x.R, x.C, x.D, x.B
        self.oR, self.oC, self.oD, self.oB = y.R, y.C, y.D, y.B
        self.K, self.stride, self.padding, self.group = kernel_size, stride, pad, group
        self.bias_term = bias_term
        self.needs_to_calc_backward_grad = True
        self.fuse_relu = False           # forward(): clamp the output at 0 (the ReLU bridge behind this layer)
        self.fuse_relu_backward = False  # backward(): input gradient times [input > 0] (the ReLU bridge in front)
        self.pool_fusion = None          # see fuse_pool_relu_backward()
        if self.iR != self.iC:
            raise ValueError("square inputs only, as in the reference")
        self.desc = capi.ConvDesc(self.iB, self.iD, self.iR, self.oD, kernel_size, stride, pad, group,
                                  int(bias_term), algo)
        m = C.c_int()
        capi.check(self.lib.cct_conv_out_size(C.byref(self.desc), C.byref(m)), "cct_conv_out_size")
        if (m.value, m.value, self.iB) != (self.oR, self.oC, self.oB):
            raise ValueError("output layer is %dx%dxB%d, convolution produces %dx%dxB%d" %
                             (self.oR, self.oC, self.oB, m.value, m.value, self.iB))
        plan = C.c_void_p()
        capi.check(self.lib.cct_conv_plan_create(self.ctx.h, C.byref(self.desc), C.byref(plan)),
                   "cct_conv_plan_create", self.ctx.h)
        self.plan = plan
        dg = self.iD // group
        self.p_model_cube = LogicalCube(self.ctx, kernel_size, kernel_size, dg, self.oD)
        self.p_model_gradient_cube = LogicalCube(self.ctx, kernel_size, kernel_size, dg, self.oD)
        self.p_bias_cube = LogicalCube(self.ctx, 1, 1, self.oD, 1) if bias_term else None
        self.p_bias_gradient_cube = LogicalCube(self.ctx, 1, 1, self.oD, 1) if bias_term else None

    # -- accessors named as in the reference
    def get_model_cube(self):
        return self.p_model_cube

    def get_bias_cube(self):
        return self.p_bias_cube

    def get_model_grad_cube(self):
        return self.p_model_gradient_cube

    def get_bias_grad_cube(self):
        return self.p_bias_gradient_cube

    def set_model_cube(self, cube):
        self.p_model_cube = cube

    def set_bias_cube(self, cube):
        self.p_bias_cube = cube

    @property
    def algo(self):
        a = C.c_int()
        capi.check(self.lib.cct_conv_plan_algo(self.plan, C.byref(a)), "cct_conv_plan_algo")
        return a.value

    @property
    def workspace_bytes(self):
        b = C.c_size_t()
        capi.check(self.lib.cct_conv_plan_workspace_bytes(self.plan, C.byref(b)), "cct_conv_plan_workspace_bytes")
        return b.value

    def forward(self):
        bias = self.p_bias_cube.ptr if self.bias_term else None
        capi.check(self.lib.cct_conv_forward(self.plan, self.p_input_layer.p_data_cube.ptr, self.p_model_cube.ptr, bias,
                                             self.p_output_layer.p_data_cube.ptr, int(self.fuse_relu)),
                   "cct_conv_forward", self.ctx.h)

    def fuse_pool_relu_backward(self, pooled_gradient_cube, max_index_cube, kernel_size, stride, pooled_data_cube=None):
        """Fold the ReLU and max-pooling bridges that follow this layer into backward(): the output gradient is
        rebuilt from the pooled tensor's gradient and the pooling indices (MaxPoolingBridge::backward then
        ReLUBridge::backward in the reference) instead of being read from p_output_layer.p_gradient_cube.  With
        `pooled_data_cube` (the pooling bridge's output, still as the forward pass wrote it when backward() runs) the
        ReLU mask is read from it instead of from this layer's much larger output: same result, fewer bytes."""
        capi.check(self.lib.cct_conv_plan_reserve_fusion(self.plan), "cct_conv_plan_reserve_fusion", self.ctx.h)
        self.pool_fusion = (pooled_gradient_cube, max_index_cube, kernel_size, stride, pooled_data_cube)

    def backward(self):
        dx = self.p_input_layer.p_gradient_cube.ptr if self.needs_to_calc_backward_grad else None
        db = self.p_bias_gradient_cube.ptr if self.bias_term else None
        x, w, dw = self.p_input_layer.p_data_cube.ptr, self.p_model_cube.ptr, self.p_model_gradient_cube.ptr
        if self.pool_fusion is None and not self.fuse_relu_backward:
            capi.check(self.lib.cct_conv_backward(self.plan, x, w, self.p_output_layer.p_gradient_cube.ptr, dx, dw, db),
                       "cct_conv_backward", self.ctx.h)
            return
        f = capi.BwdFusion(None, None, None, 0, 0, int(self.fuse_relu_backward), None)
        dy = self.p_output_layer.p_gradient_cube.ptr
        if self.pool_fusion is not None:
            dp, idx, k, s, pooled = self.pool_fusion
            f.A, f.idx, f.dP, f.pool_k, f.pool_s = self.p_output_layer.p_data_cube.ptr, idx.ptr, dp.ptr, k, s
            f.P = pooled.ptr if pooled is not None else None
            dy = None
        capi.check(self.lib.cct_conv_backward_fused(self.plan, x, w, dy, C.byref(f), dx, dw, db),
                   "cct_conv_backward_fused", self.ctx.h)

    def close(self):
        if self.plan:
            self.lib.cct_conv_plan_destroy(self.plan)
            self.plan = None
        for c in (self.p_model_cube, self.p_model_gradient_cube, self.p_bias_cube, self.p_bias_gradient_cube):
            if c is not None:
                c.free()


class FullyConnectedBridge:
    """The reference's FullyConnectedBridge (src/bridges/FullyConnectedBridge_impl.hxx:171-235, 257-330): Y = X W^T + b
    over the flattened input, weight layout [o][d][r][c].  Runs on the fully connected plan of the C ABI (tensor-core
    GEMMs that read X, W and dY in place); layers whose feature counts are not multiples of 4, and
    algo=ALGO_SIMT_FP32, run as a 1x1 convolution over the input viewed as D*R*C channels of one pixel instead.
    The output layer is B x num_output x 1 x 1.

    Fusion switches (the bridges around the layer in CaffeNet): fuse_relu clamps the output at 0; dropout_mask /
    dropout_scale (a device cube of uint32, one per output element) applies DropoutBridge's forward; on the input
    side fuse_relu_backward and input_dropout_mask / input_dropout_scale fold ReLUBridge::backward and
    DropoutBridge::backward of the bridges in front of the layer into the input gradient."""

    def __init__(self, p_input_layer, p_output_layer, bias_term=True, algo=capi.ALGO_AUTO, ctx=None):
        x, y = p_input_layer.p_data_cube, p_output_layer.p_data_cube
        self.p_input_layer, self.p_output_layer = p_input_layer, p_output_layer
        self.ctx = ctx or x.ctx
        self.lib = self.ctx.lib
        self.iR, self.iC, self.iD, self.iB = x.R, x.C, x.D, x.B
        self.oR, self.oC, self.oD, self.oB = y.R, y.C, y.D, y.B
        if (self.oR, self.oC, self.oB) != (1, 1, self.iB):
            raise ValueError("output layer must be B x num_output x 1 x 1")
        self.in_features = x.D * x.R * x.C
        self.bias_term = bias_term
        self.needs_to_calc_backward_grad = True
        self.fuse_relu = False
        self.fuse_relu_backward = False
        self.dropout_mask, self.dropout_scale = None, 1.0
        self.input_dropout_mask, self.input_dropout_scale = None, 1.0
        self.plan, self._conv = None, None
        use_plan = algo == capi.ALGO_UMMA_3XTF32 or (algo == capi.ALGO_AUTO and self.in_features % 4 == 0 and
                                                      self.oD % 4 == 0)
        if use_plan:
            plan = C.c_void_p()
            capi.check(self.lib.cct_fc_plan_create(self.ctx.h, self.iB, self.in_features, self.oD, int(bias_term),
                                                   C.byref(plan)), "cct_fc_plan_create", self.ctx.h)
            self.plan = plan
            self.p_model_cube = LogicalCube(self.ctx, x.R, x.C, x.D, self.oD)
            self.p_model_gradient_cube = LogicalCube(self.ctx, x.R, x.C, x.D, self.oD)
            self.p_bias_cube = LogicalCube(self.ctx, 1, 1, self.oD, 1) if bias_term else None
            self.p_bias_gradient_cube = LogicalCube(self.ctx, 1, 1, self.oD, 1) if bias_term else None
        else:
            dx = p_input_layer.p_gradient_cube
            k = self.in_features
            flat = Layer(LogicalCube(x.ctx, 1, 1, k, x.B, x.dtype, ptr=x.ptr),
                         LogicalCube(dx.ctx, 1, 1, k, dx.B, dx.dtype, ptr=dx.ptr) if dx is not None else None)
            self._conv = ConvolutionBridge(flat, p_output_layer, 1, 1, 0, 1, bias_term, algo, ctx)
            c = self._conv
            self.p_model_cube, self.p_model_gradient_cube = c.p_model_cube, c.p_model_gradient_cube
            self.p_bias_cube, self.p_bias_gradient_cube = c.p_bias_cube, c.p_bias_gradient_cube

    @property
    def algo(self):
        return capi.ALGO_UMMA_3XTF32 if self.plan else self._conv.algo

    def get_model_cube(self):
        return self.p_model_cube

    def get_bias_cube(self):
        return self.p_bias_cube

    def get_model_grad_cube(self):
        return self.p_model_gradient_cube

    def get_bias_grad_cube(self):
        return self.p_bias_gradient_cube

    def forward(self):
        if self._conv:
            if self.dropout_mask is not None:
                raise ValueError("dropout fusion needs the fully connected plan")
            self._conv.fuse_relu = self.fuse_relu
            self._conv.forward()
            return
        vp = C.c_void_p
        mask = self.dropout_mask.ptr if self.dropout_mask is not None else None
        capi.check(self.lib.cct_fc_forward(self.plan, vp(self.p_input_layer.p_data_cube.ptr), vp(self.p_model_cube.ptr),
                                           vp(self.p_bias_cube.ptr) if self.bias_term else None,
                                           vp(self.p_output_layer.p_data_cube.ptr), int(self.fuse_relu), mask,
                                           float(self.dropout_scale)), "cct_fc_forward", self.ctx.h)

    def backward(self):
        if self._conv:
            if self.input_dropout_mask is not None:
                raise ValueError("dropout fusion needs the fully connected plan")
            self._conv.needs_to_calc_backward_grad = self.needs_to_calc_backward_grad
            self._conv.fuse_relu_backward = self.fuse_relu_backward
            self._conv.backward()
            return
        vp = C.c_void_p
        dx = self.p_input_layer.p_gradient_cube.ptr if self.needs_to_calc_backward_grad else None
        mask = self.input_dropout_mask.ptr if self.input_dropout_mask is not None else None
        capi.check(self.lib.cct_fc_backward(self.plan, vp(self.p_input_layer.p_data_cube.ptr), vp(self.p_model_cube.ptr),
                                            vp(self.p_output_layer.p_gradient_cube.ptr), dx,
                                            vp(self.p_model_gradient_cube.ptr),
                                            vp(self.p_bias_gradient_cube.ptr) if self.bias_term else None,
                                            int(self.fuse_relu_backward), mask, float(self.input_dropout_scale)),
                   "cct_fc_backward", self.ctx.h)

    def close(self):
        if self._conv:
            self._conv.close()
            self._conv = None
            return
        if self.plan:
            self.lib.cct_fc_plan_destroy(self.plan)
            self.plan = None
        for c in (self.p_model_cube, self.p_model_gradient_cube, self.p_bias_cube, self.p_bias_gradient_cube):
            if c is not None:
                c.free()


def conv_layer(ctx, X, W, bias, dY, kernel, stride=1, pad=0, group=1, needs_dx=True, algo=capi.ALGO_AUTO, relu=False):
    """Convenience for tests: numpy in, numpy out (Y, dX, dW, db) through a ConvolutionBridge."""
    B, D, n, _ = X.shape
    o = W.shape[0]
    m = (n + 2 * pad - kernel) // stride + 1
    xin = Layer(LogicalCube.from_numpy(ctx, X), LogicalCube(ctx, n, n, D, B))
    out = Layer(LogicalCube(ctx, m, m, o, B), LogicalCube(ctx, m, m, o, B))
    br = ConvolutionBridge(xin, out, kernel, stride, pad, group, bias is not None, algo)
    br.needs_to_calc_backward_grad = needs_dx
    br.fuse_relu = relu
    br.p_model_cube.upload(W)
    if bias is not None:
        br.p_bias_cube.upload(bias)
    br.forward()
    Y = out.p_data_cube.download()
    res = [Y, None, None, None]
    if dY is not None:
        out.p_gradient_cube.upload(dY)
        br.backward()
        ctx.sync()
        res[1] = xin.p_gradient_cube.download() if needs_dx else None
        res[2] = br.p_model_gradient_cube.download()
        res[3] = br.p_bias_gradient_cube.download().reshape(-1) if bias is not None else None
    ctx.sync()
    used = br.algo
    br.close()
    for layer in (xin, out):
        layer.p_data_cube.free()
        layer.p_gradient_cube.free()
    return tuple(res) + (used,)
