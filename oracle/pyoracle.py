"""TEST INFRASTRUCTURE — ctypes access to the two CPU checkers (never imported by the product package).

`port`      : oracle/liboracle.so, the plain-C restatement (conv_oracle.c).
`reference` : oracle/_ref/libcct_ref.so, the reference's own CPU code behind ref_wrapper.cpp (None when the
              library was not built; it can only be built where the reference tree is mounted, the built file
              travels).
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_f = np.float32
_fp = C.POINTER(C.c_float)
_ip = C.POINTER(C.c_int)


def _p(a):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    if a.dtype == np.float32:
        return a.ctypes.data_as(_fp)
    if a.dtype == np.int32:
        return a.ctypes.data_as(_ip)
    raise TypeError(a.dtype)


def out_size(n, k, s, p):
    return (n + 2 * p - k) // s + 1


class Port:
    def __init__(self, path=None):
        path = path or os.path.join(HERE, "liboracle.so")
        self.lib = C.CDLL(path)
        L = self.lib
        L.oracle_conv_forward.argtypes = [_fp, _fp, _fp, _fp] + [C.c_int] * 9
        L.oracle_conv_backward.argtypes = [_fp, _fp, _fp, _fp, _fp, _fp] + [C.c_int] * 9
        L.oracle_lower_type1.argtypes = [_fp, _fp] + [C.c_int] * 6
        L.oracle_inverse_lower.argtypes = [_fp, _fp] + [C.c_int] * 6
        L.oracle_maxpool_forward.argtypes = [_fp, _fp, _ip] + [C.c_int] * 4
        L.oracle_maxpool_backward.argtypes = [_fp, _ip, _fp] + [C.c_int] * 3
        L.oracle_relu_forward.argtypes = [_fp, _fp, C.c_size_t]
        L.oracle_relu_backward.argtypes = [_fp, _fp, _fp, C.c_size_t]
        L.oracle_sgd_update.argtypes = [C.c_size_t, _fp, _fp, _fp, C.c_float, C.c_float, C.c_float]
        L.oracle_learning_rate.argtypes = [C.c_int] + [C.c_float] * 6
        L.oracle_learning_rate.restype = C.c_float

    def conv_forward(self, X, W, bias, k, s, p, g=1, acc64=False):
        B, D, n, _ = X.shape
        o = W.shape[0]
        m = out_size(n, k, s, p)
        Y = np.empty((B, o, m, m), _f)
        self.lib.oracle_conv_forward(_p(X), _p(W), _p(bias), _p(Y), B, D, n, o, k, s, p, g, int(acc64))
        return Y

    def conv_backward(self, X, W, dY, k, s, p, g=1, needs_dx=True, bias=True, acc64=False):
        B, D, n, _ = X.shape
        o = W.shape[0]
        dX = np.empty_like(X) if needs_dx else None
        dW = np.empty_like(W)
        db = np.empty((o,), _f) if bias else None
        self.lib.oracle_conv_backward(_p(X), _p(W), _p(dY), _p(dX), _p(dW), _p(db), B, D, n, o, k, s, p, g,
                                      int(acc64))
        return dX, dW, db

    def lower(self, X, k, s, p):
        B, D, n, _ = X.shape
        m = out_size(n, k, s, p)
        Dhat = np.empty((B * m * m, D * k * k), _f)
        self.lib.oracle_lower_type1(_p(X), _p(Dhat), B, D, n, k, s, p)
        return Dhat

    def inverse_lower(self, G, B, D, n, k, s, p):
        dX = np.empty((B, D, n, n), _f)
        self.lib.oracle_inverse_lower(_p(G), _p(dX), B, D, n, k, s, p)
        return dX

    def maxpool_forward(self, X, k, s):
        B, D, n, _ = X.shape
        m = (n - k) // s + 1
        Y = np.empty((B, D, m, m), _f)
        idx = np.empty((B, D, m, m), np.int32)
        self.lib.oracle_maxpool_forward(_p(X), _p(Y), _p(idx), B * D, n, k, s)
        return Y, idx

    def maxpool_backward(self, dY, idx, n):
        B, D, m, _ = dY.shape
        dX = np.empty((B, D, n, n), _f)
        self.lib.oracle_maxpool_backward(_p(dY), _p(idx), _p(dX), B * D, n, m)
        return dX

    def relu_forward(self, X):
        Y = np.empty_like(X)
        self.lib.oracle_relu_forward(_p(X), _p(Y), X.size)
        return Y

    def relu_backward(self, X, dY):
        dX = np.empty_like(X)
        self.lib.oracle_relu_backward(_p(X), _p(dY), _p(dX), X.size)
        return dX

    def sgd_update(self, w, g, h, lr, momentum, lam):
        """In place on w, g (decay is added to g, as the reference does) and h."""
        self.lib.oracle_sgd_update(w.size, _p(w), _p(g), _p(h), lr, momentum, lam)

    def learning_rate(self, policy, base_lr, gamma, it, stepsize, power=0.0, max_iter=1.0):
        pid = {"fixed": 0, "step": 1, "exp": 2, "inv": 3, "poly": 4, "sigmoid": 5}[policy]
        return float(self.lib.oracle_learning_rate(pid, base_lr, gamma, it, stepsize, power, max_iter))


class Reference:
    """The reference's compiled CPU bridges. Grouped layers are run once per channel slice."""

    def __init__(self, path=None):
        path = path or os.path.join(HERE, "_ref", "libcct_ref.so")
        self.lib = C.CDLL(path)
        L = self.lib
        L.cctref_conv_create.restype = C.c_void_p
        L.cctref_conv_create.argtypes = [C.c_int] * 10 + [C.c_float] * 3
        L.cctref_conv_destroy.argtypes = [C.c_void_p]
        L.cctref_conv_set_model.argtypes = [C.c_void_p, _fp, _fp]
        L.cctref_conv_get_model.argtypes = [C.c_void_p, _fp, _fp]
        L.cctref_conv_forward.argtypes = [C.c_void_p, _fp, _fp]
        L.cctref_conv_backward.argtypes = [C.c_void_p, _fp, _fp, _fp, _fp, C.c_int]
        L.cctref_conv_load.argtypes = [C.c_void_p, _fp, _fp]
        L.cctref_conv_step.argtypes = [C.c_void_p, C.c_int]
        L.cctref_conv_time.restype = C.c_double
        L.cctref_conv_time.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_double), C.POINTER(C.c_double)]
        L.cctref_maxpool.argtypes = [C.c_int] * 5 + [_fp, _fp, _ip, _fp, _fp]
        L.cctref_relu.argtypes = [C.c_int] * 3 + [_fp, _fp, _fp, _fp]
        L.cctref_blas_config.restype = C.c_char_p
        L.cctref_default_partitions.argtypes = [C.c_int]
        _up = C.POINTER(C.c_uint)
        for name, args in (("cctref_lrn", [C.c_int] * 4 + [C.c_float] * 2 + [_fp] * 4 + [C.c_int]),
                           ("cctref_dropout", [C.c_int] * 3 + [C.c_float, C.c_int, _fp, _fp, _up, _fp, _fp, C.c_int]),
                           ("cctref_fc", [C.c_int] * 4 + [_fp] * 8 + [C.c_int] * 2),
                           ("cctref_softmax_loss", [C.c_int] * 2 + [_fp] * 5 + [C.c_int])):
            fn = getattr(L, name, None)
            if fn is not None:  # a library built before these wrappers existed lacks them
                fn.argtypes = args
                fn.restype = C.c_double

    def hardware_concurrency(self):
        return int(self.lib.cctref_hardware_concurrency())

    def default_partitions(self, batch):
        return int(self.lib.cctref_default_partitions(batch))

    def blas_config(self):
        return self.lib.cctref_blas_config().decode()

    def conv_create(self, B, D, n, o, k, s, p, bias=True, partitions=1, needs_dx=True, lr=0.01, momentum=0.0,
                    weight_decay=0.0):
        return self.lib.cctref_conv_create(B, D, n, o, k, s, p, int(bias), partitions, int(needs_dx), lr, momentum,
                                           weight_decay)

    def conv_destroy(self, h):
        self.lib.cctref_conv_destroy(h)

    def conv_fwd_bwd(self, X, W, bias, dY, k, s, p, g=1, partitions=1, needs_dx=True, sgd=None):
        """Returns Y, dX, dW, db (and the post-SGD W, bias when sgd=(lr, momentum, weight_decay))."""
        B, D, n, _ = X.shape
        o = W.shape[0]
        m = out_size(n, k, s, p)
        Dg, og = D // g, o // g
        Y = np.empty((B, o, m, m), _f)
        dX = np.empty_like(X) if needs_dx else None
        dW = np.empty_like(W)
        db = np.empty((o,), _f) if bias is not None else None
        Wn = np.empty_like(W) if sgd else None
        bn = np.empty((o,), _f) if (sgd and bias is not None) else None
        lr, mom, wd = sgd if sgd else (0.01, 0.0, 0.0)
        for gi in range(g):
            h = self.conv_create(B, Dg, n, og, k, s, p, bias is not None, partitions, needs_dx, lr, mom, wd)
            Xs = np.ascontiguousarray(X[:, gi * Dg:(gi + 1) * Dg])
            Ws = np.ascontiguousarray(W[gi * og:(gi + 1) * og])
            bs = np.ascontiguousarray(bias[gi * og:(gi + 1) * og]) if bias is not None else None
            dYs = np.ascontiguousarray(dY[:, gi * og:(gi + 1) * og])
            Ys = np.empty((B, og, m, m), _f)
            dXs = np.empty_like(Xs) if needs_dx else None
            dWs = np.empty_like(Ws)
            dbs = np.empty((og,), _f) if bias is not None else None
            self.lib.cctref_conv_set_model(h, _p(Ws), _p(bs))
            self.lib.cctref_conv_forward(h, _p(Xs), _p(Ys))
            self.lib.cctref_conv_backward(h, _p(dYs), _p(dXs), _p(dWs), _p(dbs), int(bool(sgd)))
            Y[:, gi * og:(gi + 1) * og] = Ys
            if needs_dx:
                dX[:, gi * Dg:(gi + 1) * Dg] = dXs
            dW[gi * og:(gi + 1) * og] = dWs
            if bias is not None:
                db[gi * og:(gi + 1) * og] = dbs
            if sgd:
                Wo = np.empty_like(Ws)
                bo = np.empty((og,), _f) if bias is not None else None
                self.lib.cctref_conv_get_model(h, _p(Wo), _p(bo))
                Wn[gi * og:(gi + 1) * og] = Wo
                if bias is not None:
                    bn[gi * og:(gi + 1) * og] = bo
            self.conv_destroy(h)
        if sgd:
            return Y, dX, dW, db, Wn, bn
        return Y, dX, dW, db

    def conv_time(self, X, W, bias, dY, k, s, p, partitions, needs_dx=True, warmup=1, iters=3):
        """Median seconds (fwd+bwd, fwd, bwd) of the reference's ParallelizedBridge on host-resident data."""
        B, D, n, _ = X.shape
        o = W.shape[0]
        h = self.conv_create(B, D, n, o, k, s, p, bias is not None, partitions, needs_dx)
        self.lib.cctref_conv_set_model(h, _p(W), _p(bias))
        self.lib.cctref_conv_load(h, _p(X), _p(dY))
        tf, tb = C.c_double(), C.c_double()
        # the CPU backward permutes dY in place, so later iterations see permuted data: same work, same time
        tt = self.lib.cctref_conv_time(h, warmup, iters, C.byref(tf), C.byref(tb))
        self.conv_destroy(h)
        return tt, tf.value, tb.value

    def maxpool(self, X, k, s, dY=None):
        B, D, n, _ = X.shape
        m = (n - k) // s + 1
        Y = np.empty((B, D, m, m), _f)
        idx = np.empty((B, D, m, m), np.int32)
        dX = np.empty_like(X) if dY is not None else None
        self.lib.cctref_maxpool(B, D, n, k, s, _p(X), _p(Y), _p(idx), _p(dY), _p(dX))
        return Y, idx, dX

    def lrn(self, X, local_size, alpha, beta, dY=None, time_iters=0):
        """Y, dX (None without dY), median seconds of fwd(+bwd) when time_iters > 0."""
        B, D, n, _ = X.shape
        Y = np.empty_like(X)
        dX = np.empty_like(X) if dY is not None else None
        sec = self.lib.cctref_lrn(B, D, n, local_size, alpha, beta, _p(X), _p(Y), _p(dY), _p(dX), time_iters)
        return Y, dX, sec

    def dropout(self, X, ratio, seed, dY=None, time_iters=0):
        """Y, the mask the bridge drew (uint32, 0 / 1), dX, seconds."""
        B, D, n, _ = X.shape
        Y = np.empty_like(X)
        mask = np.empty(X.shape, np.uint32)
        dX = np.empty_like(X) if dY is not None else None
        sec = self.lib.cctref_dropout(B, D, n, ratio, seed, _p(X), _p(Y), mask.ctypes.data_as(C.POINTER(C.c_uint)),
                                      _p(dY), _p(dX), time_iters)
        return Y, mask, dX, sec

    def fill(self, kind, count, a=0.0, b=1.0, seed=1, n_batch=1):
        """`count` values from the reference's own filler: kind 0 gaussian(mean a, std b), 1 xavier over n_batch filters,
        2 bernoulli(p = a) (CPUDriver::s*_initialize, src/sched/DeviceDriver_CPU.cpp:661-699)."""
        out = np.empty(count, _f)
        self.lib.cctref_fill.argtypes = [C.c_int, C.POINTER(C.c_float), C.c_long, C.c_float, C.c_float, C.c_int, C.c_long]
        self.lib.cctref_fill.restype = None
        self.lib.cctref_fill(kind, _p(out), count, a, b, seed, n_batch)
        return out

    def fc(self, X, W, bias, dY=None, blas_threads=1, time_iters=0):
        """Y, dX, dW, db, seconds through the reference's FullyConnectedBridge."""
        B, D, n, _ = X.shape
        o = W.shape[0]
        Y = np.empty((B, o, 1, 1), _f)
        dX = np.empty_like(X) if dY is not None else None
        dW = np.empty_like(W) if dY is not None else None
        db = np.empty((o,), _f) if (dY is not None and bias is not None) else None
        sec = self.lib.cctref_fc(B, D, n, o, _p(X), _p(W), _p(bias), _p(Y), _p(dY), _p(dX), _p(dW), _p(db), blas_threads,
                                 time_iters)
        return Y, dX, dW, db, sec

    def softmax_loss(self, X, labels, time_iters=0):
        """prob, loss (summed over the batch), dX (scaled by 1 / batch), seconds."""
        B = X.shape[0]
        Cn = X.size // B
        prob, dX = np.empty_like(X), np.empty_like(X)
        loss = C.c_float()
        lab = np.ascontiguousarray(labels, dtype=_f)
        sec = self.lib.cctref_softmax_loss(B, Cn, _p(X), _p(lab), _p(prob), C.byref(loss), _p(dX), time_iters)
        return prob, float(loss.value), dX, sec

    def relu(self, X, dY=None):
        B, D, n, _ = X.shape
        Y = np.empty_like(X)
        dX = np.empty_like(X) if dY is not None else None
        self.lib.cctref_relu(B, D, n, _p(X), _p(Y), _p(dY), _p(dX))
        return Y, dX


# ---- numpy restatements of the remaining CaffeNet bridges (float64 inside, so they can serve as the "truth" side)

def np_lrn_forward(X, local_size, alpha, beta):
    """LRNBridge::forward (src/kernels/lrn.hxx:38-124): scale = 1 + alpha/size * sum of squares over the window of
    local_size channels; Y = X / scale^beta.  Returns (Y, scale) as float32."""
    X64 = X.astype(np.float64)
    B, D = X.shape[:2]
    w = local_size // 2
    sq = X64 * X64
    ssum = np.zeros_like(X64)
    for d in range(D):
        ssum[:, d] = sq[:, max(0, d - w):min(D, d + w + 1)].sum(axis=1)
    scale = 1.0 + (alpha / local_size) * ssum
    return (X64 / scale ** beta).astype(_f), scale.astype(_f)


def np_lrn_backward(X, dY, local_size, alpha, beta):
    """LRNBridge::backward (src/kernels/lrn.hxx:134-180), collected per input channel."""
    X64, dY64 = X.astype(np.float64), dY.astype(np.float64)
    B, D = X.shape[:2]
    w = local_size // 2
    sq = X64 * X64
    scale = np.ones_like(X64)
    for d in range(D):
        scale[:, d] += (alpha / local_size) * sq[:, max(0, d - w):min(D, d + w + 1)].sum(axis=1)
    t = dY64 * X64 * scale ** (-beta - 1.0)
    dX = dY64 * scale ** (-beta)
    for c in range(D):
        dX[:, c] -= 2.0 * beta * (alpha / local_size) * X64[:, c] * t[:, max(0, c - w):min(D, c + w + 1)].sum(axis=1)
    return dX.astype(_f)


def np_softmax_loss(X, labels, scale=None):
    """SoftmaxLossBridge (src/kernels/softmax.hxx:17-80): prob, summed loss, gradient (prob - onehot) * scale
    (scale defaults to 1 / batch)."""
    B = X.shape[0]
    X64 = X.reshape(B, -1).astype(np.float64)
    e = np.exp(X64 - X64.max(axis=1, keepdims=True))
    prob = e / e.sum(axis=1, keepdims=True)
    lab = labels.astype(np.int64).reshape(B)
    tiny = np.finfo(np.float32).tiny
    loss = float(-np.log(np.maximum(prob[np.arange(B), lab], tiny)).sum())
    g = prob.copy()
    g[np.arange(B), lab] -= 1.0
    g *= (1.0 / B) if scale is None else scale
    return prob.astype(_f).reshape(X.shape), loss, g.astype(_f).reshape(X.shape)


_port = None
_reference = None


def port():
    global _port
    if _port is None:
        _port = Port()
    return _port


def reference():
    """The compiled reference, or None if oracle/_ref/libcct_ref.so is not there or cannot be loaded."""
    global _reference
    if _reference is None:
        try:
            _reference = Reference()
        except OSError:
            _reference = False
    return _reference or None
