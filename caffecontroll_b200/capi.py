"""ctypes binding of include/cct_b200.h (libcct_b200.so).

There is no CPU fallback: loading fails loudly when the library has not been built, and creating a context
fails when no sm_100 device is present.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("CCT_B200_LIB") or os.path.join(HERE, "libcct_b200.so")

CCT_OK, CCT_ERR_INVALID, CCT_ERR_CUDA, CCT_ERR_NOMEM, CCT_ERR_TIMEOUT, CCT_ERR_UNSUPPORTED = range(6)
ALGO_AUTO, ALGO_SIMT_FP32, ALGO_UMMA_3XTF32 = 0, 1, 2
FILL_GAUSSIAN, FILL_XAVIER, FILL_BERNOULLI = 0, 1, 2
COMM_ID_BYTES = 128
_ERR_NAMES = {1: "CCT_ERR_INVALID", 2: "CCT_ERR_CUDA", 3: "CCT_ERR_NOMEM", 4: "CCT_ERR_TIMEOUT",
              5: "CCT_ERR_UNSUPPORTED"}

# Every symbol include/cct_b200.h declares; tests check the library exports each one.
EXPORTS = [
    "cct_ctx_create", "cct_ctx_create_on_stream", "cct_ctx_destroy", "cct_sync", "cct_last_error_string",
    "cct_device_count", "cct_malloc", "cct_free", "cct_malloc_host", "cct_free_host", "cct_memcpy_h2d",
    "cct_memcpy_d2h", "cct_memcpy_d2d", "cct_memcpy2d_d2d", "cct_memset", "cct_fill_f32", "cct_fill_random", "cct_conv_plan_create",
    "cct_conv_plan_destroy", "cct_conv_out_size", "cct_conv_plan_algo", "cct_conv_plan_workspace_bytes",
    "cct_conv_plan_enable_timing", "cct_conv_plan_last_timings", "cct_conv_forward", "cct_conv_backward", "cct_conv_backward_fused",
    "cct_conv_plan_reserve_fusion", "cct_selftest_bounded_wait", "cct_conv_forward_host", "cct_conv_backward_host", "cct_conv_weight_grad_noalloc",
    "cct_maxpool_forward", "cct_maxpool_backward", "cct_relu_forward", "cct_relu_backward",
    "cct_pool_relu_backward", "cct_sgd_step", "cct_saxpby", "cct_l1_update",
    "cct_fc_plan_create", "cct_fc_plan_destroy", "cct_fc_plan_workspace_bytes", "cct_fc_forward", "cct_fc_backward",
    "cct_fc_plan_enable_timing", "cct_fc_plan_last_timings",
    "cct_comm_unique_id", "cct_comm_init_rank", "cct_comm_destroy", "cct_comm_size", "cct_allreduce_sum_begin",
    "cct_comm_wait", "cct_allreduce_sum", "cct_allgather", "cct_reduce_scatter_sum",
    "cct_lrn_forward", "cct_lrn_backward", "cct_dropout_apply", "cct_dropout_mask", "cct_softmax_loss_forward", "cct_softmax_loss_backward",
]


class CctError(RuntimeError):
    def __init__(self, code, where, detail=""):
        self.code = code
        super().__init__("%s failed: %s%s" % (where, _ERR_NAMES.get(code, code), (" — " + detail) if detail else ""))


class BwdFusion(C.Structure):
    """cct_bwd_fusion: what cct_conv_backward_fused folds into the backward pass."""
    _fields_ = [("A", C.c_void_p), ("idx", C.c_void_p), ("dP", C.c_void_p), ("pool_k", C.c_int), ("pool_s", C.c_int),
                ("relu_mask_dx", C.c_int), ("P", C.c_void_p)]


class ConvDesc(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("batch", "in_depth", "in_size", "out_depth", "kernel", "stride", "pad",
                                        "groups", "bias_term", "algo")]


_vp = C.c_void_p
_lib = None


def load():
    """Load libcct_b200.so (raises OSError with a build hint when it is missing)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise OSError("%s not found: build it with `python -m caffecontroll_b200._build` "
                      "(there is no CPU fallback)" % LIB_PATH)
    L = C.CDLL(LIB_PATH)
    sz, i, f = C.c_size_t, C.c_int, C.c_float
    sigs = {
        "cct_ctx_create": [i, C.POINTER(_vp)],
        "cct_ctx_create_on_stream": [i, _vp, C.POINTER(_vp)],
        "cct_ctx_destroy": [_vp],
        "cct_sync": [_vp],
        "cct_device_count": [C.POINTER(i)],
        "cct_malloc": [_vp, sz, C.POINTER(_vp)],
        "cct_free": [_vp, _vp],
        "cct_malloc_host": [_vp, sz, C.POINTER(_vp)],
        "cct_free_host": [_vp, _vp],
        "cct_memcpy_h2d": [_vp, _vp, _vp, sz],
        "cct_memcpy_d2h": [_vp, _vp, _vp, sz],
        "cct_memcpy_d2d": [_vp, _vp, _vp, sz],
        "cct_memcpy2d_d2d": [_vp, _vp, sz, _vp, sz, sz, sz],
        "cct_memset": [_vp, _vp, i, sz],
        "cct_fill_f32": [_vp, _vp, sz, f],
        "cct_fill_random": [_vp, _vp, sz, i, f, f, C.c_long],
        "cct_conv_plan_create": [_vp, C.POINTER(ConvDesc), C.POINTER(_vp)],
        "cct_conv_plan_destroy": [_vp],
        "cct_conv_out_size": [C.POINTER(ConvDesc), C.POINTER(i)],
        "cct_conv_plan_algo": [_vp, C.POINTER(i)],
        "cct_conv_plan_workspace_bytes": [_vp, C.POINTER(sz)],
        "cct_conv_plan_enable_timing": [_vp, i],
        "cct_conv_plan_last_timings": [_vp, C.POINTER(C.c_float)],
        "cct_conv_forward": [_vp, _vp, _vp, _vp, _vp, i],
        "cct_conv_backward": [_vp, _vp, _vp, _vp, _vp, _vp, _vp],
        "cct_conv_backward_fused": [_vp, _vp, _vp, _vp, C.POINTER(BwdFusion), _vp, _vp, _vp],
        "cct_conv_plan_reserve_fusion": [_vp],
        "cct_selftest_bounded_wait": [_vp, C.c_longlong],
        "cct_conv_forward_host": [_vp, _vp, _vp, _vp, _vp, i],
        "cct_conv_backward_host": [_vp, _vp, _vp, _vp, _vp, _vp, _vp],
        "cct_conv_weight_grad_noalloc": [_vp, C.POINTER(ConvDesc), _vp, _vp, _vp, _vp],
        "cct_maxpool_forward": [_vp, _vp, _vp, _vp, i, i, i, i],
        "cct_maxpool_backward": [_vp, _vp, _vp, _vp, i, i, i, i],
        "cct_relu_forward": [_vp, _vp, _vp, sz],
        "cct_relu_backward": [_vp, _vp, _vp, _vp, sz],
        "cct_pool_relu_backward": [_vp, _vp, _vp, _vp, _vp, i, i, i, i],
        "cct_sgd_step": [_vp, sz, _vp, _vp, _vp, f, f, f],
        "cct_saxpby": [_vp, sz, f, _vp, f, _vp],
        "cct_l1_update": [_vp, sz, _vp, f, _vp],
        "cct_comm_unique_id": [C.c_char_p],
        "cct_comm_init_rank": [_vp, i, i, C.c_char_p, C.POINTER(_vp)],
        "cct_comm_destroy": [_vp],
        "cct_comm_size": [_vp, C.POINTER(i), C.POINTER(i)],
        "cct_allreduce_sum_begin": [_vp, _vp, sz],
        "cct_comm_wait": [_vp],
        "cct_allreduce_sum": [_vp, _vp, sz],
        "cct_allgather": [_vp, _vp, _vp, sz],
        "cct_reduce_scatter_sum": [_vp, _vp, _vp, sz],
        "cct_lrn_forward": [_vp, _vp, _vp, _vp, i, i, i, i, f, f],
        "cct_lrn_backward": [_vp, _vp, _vp, _vp, _vp, _vp, i, i, i, i, f, f],
        "cct_dropout_apply": [_vp, _vp, _vp, f, _vp, sz],
        "cct_dropout_mask": [_vp, _vp, sz, f, C.c_uint64, C.c_uint64],
        "cct_softmax_loss_forward": [_vp, _vp, _vp, _vp, _vp, _vp, i, i],
        "cct_softmax_loss_backward": [_vp, _vp, _vp, _vp, i, i, f],
        "cct_fc_plan_create": [_vp, i, i, i, i, C.POINTER(_vp)],
        "cct_fc_plan_destroy": [_vp],
        "cct_fc_plan_workspace_bytes": [_vp, C.POINTER(sz)],
        "cct_fc_forward": [_vp, _vp, _vp, _vp, _vp, i, _vp, f],
        "cct_fc_backward": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, i, _vp, f],
        "cct_fc_plan_enable_timing": [_vp, i],
        "cct_fc_plan_last_timings": [_vp, C.POINTER(C.c_float)],
    }
    for name, args in sigs.items():
        fn = getattr(L, name)
        fn.argtypes = args
        fn.restype = C.c_int
    L.cct_last_error_string.argtypes = [_vp]
    L.cct_last_error_string.restype = C.c_char_p
    _lib = L
    return L


def check(code, where, ctx=None):
    if code != CCT_OK:
        detail = ""
        if ctx:
            detail = load().cct_last_error_string(ctx).decode(errors="replace")
        raise CctError(code, where, detail)
