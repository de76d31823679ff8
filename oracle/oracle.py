"""NumPy-level access to the CPU restatement in oracle/oracle_*.c.

TEST INFRASTRUCTURE ONLY: the checker that the CUDA path is compared with.
Only tests/, the smoke check and the benchmark's CPU-baseline leg import this
module; the product package never does.

Parity status: pinned against the reference's own compiled CPU functions
(oracle/ref.py) and the fixtures in tests/golden/ — see the header of
oracle_quant.c; the fp32 summation order of the contractions is unpinned
(Eigen is not available), see oracle_contract.c.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None

_f32p = ctypes.POINTER(ctypes.c_float)
_i64p = ctypes.POINTER(ctypes.c_int64)


def build(force=False):
    """Compile liboracle.so with the flags of oracle/Makefile (target `oracle`)."""
    srcs = sorted(os.path.join(_HERE, f) for f in os.listdir(_HERE) if f.startswith("oracle_") and f.endswith(".c"))
    if not force and os.path.exists(LIB_PATH) and all(
            os.path.getmtime(LIB_PATH) >= os.path.getmtime(s) for s in srcs):
        return LIB_PATH
    subprocess.check_call(["gcc", "-O2", "-fPIC", "-shared", "-fno-fast-math", "-ffp-contract=off",
                           "-o", LIB_PATH] + srcs + ["-lm"])
    return LIB_PATH


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.oracle_min_max_quantize.restype = ctypes.c_int
        _lib.oracle_convolution.restype = ctypes.c_int
        _lib.oracle_pow2_thresholds.restype = ctypes.c_int
        _lib.oracle_pool_out.restype = ctypes.c_int
    return _lib


def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return a.ctypes.data_as(_f32p) if a is not None else None


def _shape(s):
    return (ctypes.c_int64 * max(1, len(s)))(*[int(v) for v in s])


def fixed_point_quantize(x, sign=True, n=8, delta=2.0 ** -4):
    x = _f(x)
    y = np.empty_like(x)
    lib().oracle_fixed_point_quantize(_p(x), _p(y), ctypes.c_int64(x.size), int(sign), int(n),
                                      ctypes.c_float(delta))
    return y


def pow2_quantize(x, sign=True, with_zero=True, n=8, m=1):
    x = _f(x)
    y = np.empty_like(x)
    lib().oracle_pow2_quantize(_p(x), _p(y), ctypes.c_int64(x.size), int(sign), int(with_zero), int(n), int(m))
    return y


def pow2_constants(sign, with_zero, n, m):
    a, b, c = ctypes.c_float(), ctypes.c_float(), ctypes.c_float()
    lib().oracle_pow2_constants(int(sign), int(with_zero), int(n), int(m), ctypes.byref(a), ctypes.byref(b),
                                ctypes.byref(c))
    return a.value, b.value, c.value


def pow2_thresholds():
    """(table[254] of uint32 mantissa cuts for e = -126..127, n_non_monotone)."""
    t = np.zeros(254, dtype=np.uint32)
    bad = lib().oracle_pow2_thresholds(t.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32)))
    return t, bad


def min_max_quantize(x, qr_min, qr_max, ql_min, ql_max, decay=0.999, x_min_max=False, ema=False, eps=0.01):
    """Returns (y, qr_min_after, qr_max_after, scale)."""
    x = _f(x)
    qr_min, qr_max = _f(qr_min).copy(), _f(qr_max).copy()
    ql_min, ql_max = _f(ql_min), _f(ql_max)
    qshape = qr_min.shape
    if len(qshape) != x.ndim:
        raise ValueError("q tensors must have the same ndim as x")
    y = np.empty_like(x)
    scale = np.empty_like(qr_min)
    rc = lib().oracle_min_max_quantize(_p(x), _shape(x.shape), x.ndim, _p(qr_min), _p(qr_max), _p(ql_min),
                                       _p(ql_max), _shape(qshape), ctypes.c_float(decay), int(x_min_max),
                                       int(ema), ctypes.c_float(eps), _p(y), _p(scale))
    if rc != 0:
        raise ValueError("oracle_min_max_quantize: bad shapes")
    return y, qr_min, qr_max, scale


def sign(x, alpha=1.0):
    x = _f(x)
    y = np.empty_like(x)
    lib().oracle_sign(_p(x), _p(y), ctypes.c_int64(x.size), ctypes.c_float(alpha))
    return y


def binarize_columns(w2d, quantize_zero_to=1.0):
    """BinaryWeightAffine weight step: (wb, alpha[cols], scaled)."""
    w = _f(w2d)
    r, c = w.shape
    wb, sc, al = np.empty_like(w), np.empty_like(w), np.empty(c, np.float32)
    lib().oracle_binarize_columns(_p(w), ctypes.c_int64(r), ctypes.c_int64(c), ctypes.c_float(quantize_zero_to),
                                  _p(wb), _p(al), _p(sc))
    return wb, al, sc


def binarize_rows(w2d, quantize_zero_to=1.0):
    """BinaryWeightConvolution weight step: (wb, alpha[rows], scaled)."""
    w = _f(w2d)
    r, c = w.shape
    wb, sc, al = np.empty_like(w), np.empty_like(w), np.empty(r, np.float32)
    lib().oracle_binarize_rows(_p(w), ctypes.c_int64(r), ctypes.c_int64(c), ctypes.c_float(quantize_zero_to),
                               _p(wb), _p(al), _p(sc))
    return wb, al, sc


def affine(x, w, b=None, base_axis=1, f64=False):
    x, w = _f(x), _f(w)
    M = int(np.prod(x.shape[:base_axis]))
    K = x.size // M
    N = w.size // w.shape[0]
    if w.shape[0] != K:
        raise ValueError("affine: size of input and weights mismatch")
    b = _f(b).reshape(-1) if b is not None else None
    out_shape = x.shape[:base_axis] + w.shape[1:]
    if f64:
        y = np.empty((M, N), np.float64)
        lib().oracle_affine_f64(_p(x), _p(w), _p(b), ctypes.c_int64(M), ctypes.c_int64(K), ctypes.c_int64(N),
                                y.ctypes.data_as(ctypes.POINTER(ctypes.c_double)))
    else:
        y = np.empty((M, N), np.float32)
        lib().oracle_affine(_p(x), _p(w), _p(b), ctypes.c_int64(M), ctypes.c_int64(K), ctypes.c_int64(N), _p(y))
    return y.reshape(out_shape)


def conv_out_shape(xshape, wshape, pad, stride, dilation):
    N, C, H, W = xshape
    Ko, _, kh, kw = wshape
    Ho = (H + 2 * pad[0] - (dilation[0] * (kh - 1) + 1)) // stride[0] + 1
    Wo = (W + 2 * pad[1] - (dilation[1] * (kw - 1) + 1)) // stride[1] + 1
    return (N, Ko, Ho, Wo)


def convolution(x, w, b=None, pad=(0, 0), stride=(1, 1), dilation=(1, 1), group=1, f64=False):
    x, w = _f(x), _f(w)
    N, C, H, W = x.shape
    Ko, Cg, kh, kw = w.shape
    oshape = conv_out_shape(x.shape, w.shape, pad, stride, dilation)
    b = _f(b) if b is not None else None
    y = np.empty(oshape, np.float64 if f64 else np.float32)
    rc = lib().oracle_convolution(
        _p(x), _p(w), _p(b), N, C, H, W, Ko, kh, kw, pad[0], pad[1], stride[0], stride[1], dilation[0],
        dilation[1], group, None if f64 else _p(y), int(f64),
        y.ctypes.data_as(ctypes.POINTER(ctypes.c_double)) if f64 else None)
    if rc != 0:
        raise ValueError("oracle_convolution: invalid configuration")
    return y


def binary_weight_affine(x, w, b=None, base_axis=1, quantize_zero_to=1.0):
    """Returns (y, wb, alpha) like binary_weight_affine.cpp:75-122."""
    w = _f(w)
    w2 = w.reshape(w.shape[0], -1)
    wb, al, sc = binarize_columns(w2, quantize_zero_to)
    y = affine(x, sc.reshape(w.shape), b, base_axis)
    return y, wb.reshape(w.shape), al


def binary_connect_affine(x, w, b=None, base_axis=1, quantize_zero_to=1.0):
    w = _f(w)
    wb = sign(w, quantize_zero_to)
    return affine(x, wb, b, base_axis), wb


def binary_weight_convolution(x, w, b=None, pad=(0, 0), stride=(1, 1), dilation=(1, 1), group=1,
                              quantize_zero_to=1.0):
    w = _f(w)
    wb, al, sc = binarize_rows(w.reshape(w.shape[0], -1), quantize_zero_to)
    y = convolution(x, sc.reshape(w.shape), b, pad, stride, dilation, group)
    return y, wb.reshape(w.shape), al


def binary_connect_convolution(x, w, b=None, pad=(0, 0), stride=(1, 1), dilation=(1, 1), group=1,
                               quantize_zero_to=1.0):
    w = _f(w)
    wb = sign(w, quantize_zero_to)
    return convolution(x, wb, b, pad, stride, dilation, group), wb


def batch_norm_inference(x, beta, gamma, mean, var, eps=1e-5):
    x = _f(x)
    N, C = x.shape[:2]
    S = x.size // (N * C)
    y = np.empty_like(x)
    lib().oracle_batch_norm_inference(_p(x), _p(_f(beta).reshape(-1)), _p(_f(gamma).reshape(-1)),
                                      _p(_f(mean).reshape(-1)), _p(_f(var).reshape(-1)), ctypes.c_int64(N),
                                      ctypes.c_int64(C), ctypes.c_int64(S), ctypes.c_float(eps), _p(y))
    return y


def relu(x):
    x = _f(x)
    y = np.empty_like(x)
    lib().oracle_relu(_p(x), _p(y), ctypes.c_int64(x.size))
    return y


def add2(a, b):
    a, b = _f(a), _f(b)
    y = np.empty_like(a)
    lib().oracle_add2(_p(a), _p(b), _p(y), ctypes.c_int64(a.size))
    return y


def max_pooling(x, kernel, stride, ignore_border=True, pad=(0, 0)):
    x = _f(x)
    H, W = x.shape[-2:]
    maps = x.size // (H * W)
    Ho = lib().oracle_pool_out(H, kernel[0], stride[0], pad[0], int(ignore_border))
    Wo = lib().oracle_pool_out(W, kernel[1], stride[1], pad[1], int(ignore_border))
    y = np.empty(x.shape[:-2] + (Ho, Wo), np.float32)
    lib().oracle_max_pooling(_p(x), ctypes.c_int64(maps), H, W, kernel[0], kernel[1], stride[0], stride[1], pad[0],
                             pad[1], int(ignore_border), _p(y))
    return y


def global_average_pooling(x):
    x = _f(x)
    N, C = x.shape[:2]
    S = x.size // (N * C)
    y = np.empty((N, C, 1, 1), np.float32)
    lib().oracle_global_average_pooling(_p(x), ctypes.c_int64(N * C), ctypes.c_int64(S), _p(y))
    return y


def batch_norm_batch(x, beta, gamma, rmean, rvar, eps=1e-5, decay_rate=0.9, update=True):
    """Batch-statistics BatchNormalization. Returns (y, batch mean, batch var, running mean after, running var after)."""
    x = _f(x)
    N, C = x.shape[:2]
    S = x.size // (N * C)
    y = np.empty_like(x)
    m, v = np.empty(C, np.float32), np.empty(C, np.float32)
    rm, rv = _f(rmean).reshape(-1).copy(), _f(rvar).reshape(-1).copy()
    lib().oracle_batch_norm_batch(_p(x), _p(_f(beta).reshape(-1)) if beta is not None else None,
                                  _p(_f(gamma).reshape(-1)) if gamma is not None else None, _p(rm), _p(rv),
                                  ctypes.c_int64(N), ctypes.c_int64(C), ctypes.c_int64(S), ctypes.c_float(eps),
                                  ctypes.c_float(decay_rate), int(update), _p(y), _p(m), _p(v))
    return y, m, v, rm, rv


def _grad_buffer(like, accum, init):
    g = np.zeros(like, np.float32) if init is None else _f(init).reshape(like).copy()
    return g


def batch_norm_backward(x, dy, gamma, mean, var, eps=1e-5, batch_stat=True, dmean=None, dvar=None,
                        propagate_down=(True, True, True), accum=(False, False, False), grads=(None, None, None)):
    """Returns (dx, dbeta, dgamma); mean / var are the batch statistics (batch_stat) or the running ones."""
    x, dy = _f(x), _f(dy)
    N, C = x.shape[:2]
    S = x.size // (N * C)
    dx = _grad_buffer(x.shape, accum[0], grads[0])
    db = _grad_buffer((C,), accum[1], grads[1])
    dg = _grad_buffer((C,), accum[2], grads[2])
    g = _p(_f(gamma).reshape(-1)) if gamma is not None else None
    common = (ctypes.c_int64(N), ctypes.c_int64(C), ctypes.c_int64(S), ctypes.c_float(eps),
              _p(dx) if propagate_down[0] else None, int(accum[0]), _p(db) if propagate_down[1] else None,
              int(accum[1]), _p(dg) if propagate_down[2] else None, int(accum[2]))
    m, v = _f(mean).reshape(-1), _f(var).reshape(-1)
    if batch_stat:
        lib().oracle_batch_norm_batch_backward(_p(x), _p(dy), g, _p(m), _p(v),
                                               _p(_f(dmean).reshape(-1)) if dmean is not None else None,
                                               _p(_f(dvar).reshape(-1)) if dvar is not None else None, *common)
    else:
        lib().oracle_batch_norm_global_backward(_p(x), _p(dy), g, _p(m), _p(v), *common)
    return dx, db, dg


def relu_backward(y, dy, accum=False, dx=None):
    y, dy = _f(y), _f(dy)
    g = _grad_buffer(y.shape, accum, dx)
    lib().oracle_relu_backward(_p(y), _p(dy), _p(g), ctypes.c_int64(y.size), int(accum))
    return g


def add2_backward(dy, accum=False, dx=None):
    dy = _f(dy)
    g = _grad_buffer(dy.shape, accum, dx)
    lib().oracle_add2_backward(_p(dy), _p(g), ctypes.c_int64(dy.size), int(accum))
    return g


def global_average_pooling_backward(xshape, dy, accum=False, dx=None):
    dy = _f(dy)
    N, C = xshape[:2]
    S = int(np.prod(xshape[2:]))
    g = _grad_buffer(tuple(xshape), accum, dx)
    lib().oracle_global_average_pooling_backward(_p(dy), _p(g), ctypes.c_int64(N * C), ctypes.c_int64(S), int(accum))
    return g


def max_pooling_backward(x, dy, kernel, stride, ignore_border=True, pad=(0, 0), accum=False, dx=None):
    x, dy = _f(x), _f(dy)
    H, W = x.shape[-2:]
    maps = x.size // (H * W)
    g = _grad_buffer(x.shape, accum, dx)
    lib().oracle_max_pooling_backward(_p(x), _p(dy), _p(g), ctypes.c_int64(maps), H, W, kernel[0], kernel[1],
                                      stride[0], stride[1], pad[0], pad[1], int(ignore_border), int(accum))
    return g


# Backward passes -------------------------------------------------------------

def fixed_point_quantize_backward(x, dy, sign=True, n=8, delta=2.0 ** -4, ste_fine_grained=True, accum=False,
                                  dx=None):
    x, dy = _f(x), _f(dy)
    g = np.zeros_like(x) if dx is None else _f(dx).copy().reshape(x.shape)
    lib().oracle_fixed_point_quantize_backward(_p(x), _p(dy), _p(g), ctypes.c_int64(x.size), int(sign), int(n),
                                               ctypes.c_float(delta), int(ste_fine_grained), int(accum))
    return g


def pow2_quantize_backward(x, dy, sign=True, with_zero=True, n=8, m=1, ste_fine_grained=True, accum=False, dx=None):
    x, dy = _f(x), _f(dy)
    g = np.zeros_like(x) if dx is None else _f(dx).copy().reshape(x.shape)
    lib().oracle_pow2_quantize_backward(_p(x), _p(dy), _p(g), ctypes.c_int64(x.size), int(sign), int(with_zero),
                                        int(n), int(m), int(ste_fine_grained), int(accum))
    return g


def min_max_quantize_backward(x, qr_min, qr_max, ql_min, ql_max, dy, x_min_max=False, ema=False,
                              ste_fine_grained=True, propagate_down=(True, True, True),
                              accum=(False, False, False), grads=(None, None, None)):
    """qr_min / qr_max are the values the forward left behind. Returns
    (dx, g_qr_min, g_qr_max)."""
    x, dy = _f(x), _f(dy)
    qr_min, qr_max, ql_min, ql_max = _f(qr_min), _f(qr_max), _f(ql_min), _f(ql_max)
    gx = np.zeros_like(x) if grads[0] is None else _f(grads[0]).copy().reshape(x.shape)
    gmin = np.zeros_like(qr_min) if grads[1] is None else _f(grads[1]).copy().reshape(qr_min.shape)
    gmax = np.zeros_like(qr_min) if grads[2] is None else _f(grads[2]).copy().reshape(qr_min.shape)
    pd = (ctypes.c_int32 * 3)(*[int(bool(v)) for v in propagate_down])
    ac = (ctypes.c_int32 * 3)(*[int(bool(v)) for v in accum])
    L = lib()
    L.oracle_min_max_quantize_backward.restype = ctypes.c_int
    rc = L.oracle_min_max_quantize_backward(_p(x), _shape(x.shape), x.ndim, _p(qr_min), _p(qr_max), _p(ql_min),
                                            _p(ql_max), _shape(qr_min.shape), _p(dy), int(x_min_max), int(ema),
                                            int(ste_fine_grained), pd, ac, _p(gx), _p(gmin), _p(gmax))
    if rc != 0:
        raise ValueError("oracle_min_max_quantize_backward: bad shapes")
    return gx, gmin, gmax


def affine_backward(x, w, dy, base_axis=1, propagate_down=(True, True, True), accum=(False, False, False),
                    grads=(None, None, None), f64=False):
    """Affine::backward_impl (affine.cpp:98-138). Returns (dx, dw, db); entries
    whose propagate_down flag is false come back as the initial buffers."""
    x, w, dy = _f(x), _f(w), _f(dy)
    M = int(np.prod(x.shape[:base_axis]))
    K = x.size // M
    N = w.size // w.shape[0]
    shapes = (x.shape, w.shape, w.shape[1:])
    g = [np.zeros(s, np.float32) if b is None else _f(b).copy().reshape(s) for s, b in zip(shapes, grads)]
    lib().oracle_affine_backward(_p(x), _p(w), _p(dy), _p(g[0]) if propagate_down[0] else None,
                                 _p(g[1]) if propagate_down[1] else None, _p(g[2]) if propagate_down[2] else None,
                                 ctypes.c_int64(M), ctypes.c_int64(K), ctypes.c_int64(N), int(accum[0]),
                                 int(accum[1]), int(accum[2]), int(f64))
    return tuple(g)


def binary_weight_affine_backward(x, w, dy, base_axis=1, quantize_zero_to=1.0, **kw):
    """binary_weight_affine.cpp:124-146: affine backward against wb * alpha; the
    weight gradient passes straight through Sign to the float weights."""
    w = _f(w)
    _, _, sc = binarize_columns(w.reshape(w.shape[0], -1), quantize_zero_to)
    return affine_backward(x, sc.reshape(w.shape), dy, base_axis, **kw)


def binary_connect_affine_backward(x, w, dy, base_axis=1, quantize_zero_to=1.0, **kw):
    """binary_connect_affine.cpp:73-93."""
    return affine_backward(x, sign(_f(w), quantize_zero_to), dy, base_axis, **kw)


def convolution_backward(x, w, dy, pad=(0, 0), stride=(1, 1), dilation=(1, 1), group=1,
                         propagate_down=(True, True, True), accum=(False, False, False), grads=(None, None, None),
                         f64=False):
    """Convolution::backward_impl (convolution.cpp:199-300), 2-D NCHW. Returns (dx, dw, db)."""
    x, w, dy = _f(x), _f(w), _f(dy)
    N, C, H, W = x.shape
    Ko, _, kh, kw = w.shape
    shapes = (x.shape, w.shape, (Ko,))
    g = [np.zeros(s, np.float32) if b is None else _f(b).copy().reshape(s) for s, b in zip(shapes, grads)]
    L = lib()
    L.oracle_convolution_backward.restype = ctypes.c_int
    rc = L.oracle_convolution_backward(_p(x), _p(w), _p(dy), _p(g[0]) if propagate_down[0] else None,
                                       _p(g[1]) if propagate_down[1] else None,
                                       _p(g[2]) if propagate_down[2] else None, N, C, H, W, Ko, kh, kw, pad[0],
                                       pad[1], stride[0], stride[1], dilation[0], dilation[1], group, int(accum[0]),
                                       int(accum[1]), int(accum[2]), int(f64))
    if rc != 0:
        raise ValueError("oracle_convolution_backward: invalid configuration")
    return tuple(g)


def binary_weight_convolution_backward(x, w, dy, pad=(0, 0), stride=(1, 1), dilation=(1, 1), group=1,
                                       quantize_zero_to=1.0, **kw):
    """binary_weight_convolution.cpp:119-146: convolution backward against wb * alpha."""
    w = _f(w)
    _, _, sc = binarize_rows(w.reshape(w.shape[0], -1), quantize_zero_to)
    return convolution_backward(x, sc.reshape(w.shape), dy, pad, stride, dilation, group, **kw)


def binary_connect_convolution_backward(x, w, dy, pad=(0, 0), stride=(1, 1), dilation=(1, 1), group=1,
                                        quantize_zero_to=1.0, **kw):
    """binary_connect_convolution.cpp:82-104."""
    return convolution_backward(x, sign(_f(w), quantize_zero_to), dy, pad, stride, dilation, group, **kw)


# Sibling quantization functions -------------------------------------------------

def binary_sigmoid(x):
    x = _f(x)
    y = np.empty_like(x)
    lib().oracle_binary_act(_p(x), _p(y), ctypes.c_int64(x.size), 0)
    return y


def binary_tanh(x):
    x = _f(x)
    y = np.empty_like(x)
    lib().oracle_binary_act(_p(x), _p(y), ctypes.c_int64(x.size), 1)
    return y


def _binary_act_backward(x, dy, tanh_like, accum, dx):
    x, dy = _f(x), _f(dy)
    g = np.zeros_like(x) if dx is None else _f(dx).copy().reshape(x.shape)
    lib().oracle_binary_act_backward(_p(x), _p(dy), _p(g), ctypes.c_int64(x.size), int(tanh_like), int(accum))
    return g


def binary_sigmoid_backward(x, dy, accum=False, dx=None):
    return _binary_act_backward(x, dy, False, accum, dx)


def binary_tanh_backward(x, dy, accum=False, dx=None):
    return _binary_act_backward(x, dy, True, accum, dx)


def quantize_linear(x, scale, zero_point, round_mode="HALF_AWAY_FROM_ZERO", narrow_range=False, dtype=1):
    """Returns (y, zero_point_after)."""
    x, scale, zp = _f(x), _f(scale), _f(zero_point).copy()
    y = np.empty_like(x)
    L = lib()
    L.oracle_quantize_linear.restype = ctypes.c_int
    rc = L.oracle_quantize_linear(_p(x), _shape(x.shape), x.ndim, _p(scale), _shape(scale.shape), _p(zp),
                                  _shape(zp.shape), _p(y), int(round_mode == "HALF_TO_EVEN"), int(narrow_range),
                                  int(dtype))
    if rc != 0:
        raise ValueError("oracle_quantize_linear: dtype must be 1 (BYTE) or 2 (UBYTE)")
    return y, zp


def dequantize_linear(x, scale, zero_point):
    x, scale, zp = _f(x), _f(scale), _f(zero_point)
    y = np.empty_like(x)
    lib().oracle_dequantize_linear(_p(x), _shape(x.shape), x.ndim, _p(scale), _shape(scale.shape), _p(zp),
                                   _shape(zp.shape), _p(y))
    return y


def _linear_scale_backward(dy, scale, divide, accum, dx):
    dy, scale = _f(dy), _f(scale)
    g = np.zeros_like(dy) if dx is None else _f(dx).copy().reshape(dy.shape)
    lib().oracle_linear_scale_backward(_p(dy), _shape(dy.shape), dy.ndim, _p(scale), _shape(scale.shape), _p(g),
                                       int(divide), int(accum))
    return g


def quantize_linear_backward(dy, scale, accum=False, dx=None):
    return _linear_scale_backward(dy, scale, True, accum, dx)


def dequantize_linear_backward(dy, scale, accum=False, dx=None):
    return _linear_scale_backward(dy, scale, False, accum, dx)


def prune(x, rate=0.9):
    x = _f(x)
    y = np.empty_like(x)
    lib().oracle_prune(_p(x), _p(y), ctypes.c_int64(x.size), ctypes.c_float(rate))
    return y


# Incremental network quantization ---------------------------------------------

class INQState:
    """The weights' state a function instance of INQAffine keeps across forward passes."""

    def __init__(self, shape):
        self.old_w = np.zeros(shape, np.float32)
        self.old_ind = np.zeros(shape, np.int32)
        self.counter = 0


def inq_update(w, ind, state, num_bits, inq_iterations, selection_algorithm="largest_abs", draws=None):
    """One forward pass's weight update (inq_affine.cpp:82-203). Returns (weights after, indicators after);
    `state` advances. selection_algorithm="random" needs the Bernoulli draws of this pass in `draws`."""
    w = _f(w).copy()
    ind = np.ascontiguousarray(ind, np.int32).copy()
    trigger = 0
    if state.counter in list(inq_iterations):
        trigger = 2 if list(inq_iterations)[-1] == state.counter else (1 if selection_algorithm == "largest_abs" else 3)
    d = np.ascontiguousarray(draws if draws is not None else [0], np.int32)
    lib().oracle_inq_update(_p(w), ind.ctypes.data_as(ctypes.c_void_p), _p(state.old_w),
                            state.old_ind.ctypes.data_as(ctypes.c_void_p), ctypes.c_int64(w.size), int(num_bits),
                            trigger, d.ctypes.data_as(ctypes.c_void_p))
    state.counter += 1
    return w, ind


def inq_affine(x, w, ind, b, state, base_axis=1, num_bits=4, inq_iterations=(), selection_algorithm="largest_abs",
               draws=None):
    """INQAffine forward: returns (y, weights after, indicators after)."""
    w2, ind2 = inq_update(w, ind, state, num_bits, inq_iterations, selection_algorithm, draws)
    return affine(x, w2, b, base_axis), w2, ind2


def inq_convolution(x, w, ind, b, state, pad=(0, 0), stride=(1, 1), dilation=(1, 1), group=1, num_bits=4,
                    inq_iterations=(), selection_algorithm="largest_abs", draws=None):
    """INQConvolution forward (inq_convolution.cpp:86-204, the same update around Convolution)."""
    w2, ind2 = inq_update(w, ind, state, num_bits, inq_iterations, selection_algorithm, draws)
    return convolution(x, w2, b, pad, stride, dilation, group), w2, ind2
