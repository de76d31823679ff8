"""ctypes access to the reference's own CPU functions (oracle/_ref/libnnabla_ref.so).

TEST INFRASTRUCTURE ONLY. The library is the reference's C++ runtime and
hot-path functions compiled from the reference checkout by oracle/Makefile
(target `ref`); this module calls them through the C ABI in
oracle/ref_shim/ref_capi.cpp. It is used to pin the C restatement in
oracle/, to generate tests/golden/ fixtures and as bench.py's timed CPU
baseline. The product package never imports it.
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libnnabla_ref.so")


class _Tensor(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("ndim", ctypes.c_int32),
                ("shape", ctypes.c_int64 * 8)]


_lib = None


def available():
    return os.path.exists(LIB_PATH)


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.nbref_last_error.restype = ctypes.c_char_p
        _lib.nbref_forward.restype = ctypes.c_int
    return _lib


def forward(op, scalars, ivecs, inputs, n_out=1, repeat=1):
    """Run reference function `op` on the "cpu:float" context.

    scalars: constructor scalars in order; ivecs: constructor vector<int>
    arguments in order; inputs: list of float32 arrays (None entries are
    dropped, mirroring optional trailing inputs such as bias).
    Returns (outputs, inputs_after, forward_seconds). inputs_after holds the
    input buffers after the call because several functions write them.
    """
    L = lib()
    ins = [np.ascontiguousarray(a, dtype=np.float32).copy() for a in inputs if a is not None]
    s = (ctypes.c_double * max(1, len(scalars)))(*[float(v) for v in scalars])
    flat = [int(v) for vec in ivecs for v in vec]
    iv = (ctypes.c_int32 * max(1, len(flat)))(*flat)
    ivl = (ctypes.c_int32 * max(1, len(ivecs)))(*[len(v) for v in ivecs])
    tin = (_Tensor * len(ins))()
    for t, a in zip(tin, ins):
        t.data = a.ctypes.data
        t.ndim = a.ndim
        for d, n in enumerate(a.shape):
            t.shape[d] = n
    tout = (_Tensor * n_out)()
    secs = ctypes.c_double(0.0)

    def call(mode):
        rc = L.nbref_forward(op.encode(), s, len(scalars), iv, ivl, len(ivecs),
                             tin, len(ins), tout, n_out, mode, repeat,
                             ctypes.byref(secs))
        if rc != 0:
            raise RuntimeError(L.nbref_last_error().decode())

    call(0)
    outs = []
    for t in tout:
        shape = tuple(t.shape[d] for d in range(t.ndim))
        a = np.empty(shape, dtype=np.float32)
        t.data = a.ctypes.data
        outs.append(a)
    call(1)
    return outs, ins, secs.value


def backward(op, scalars, ivecs, inputs, out_grads, propagate_down, accum=None, in_grads=None):
    """Setup + forward + Function::backward of reference function `op`.

    inputs: float32 arrays (no None entries); out_grads: gradient arriving at
    each output; propagate_down / accum: one flag per input; in_grads: the
    initial gradient buffers of the inputs (zeros when omitted). Returns
    (in_grads_after, outputs, inputs_after)."""
    L = lib()
    L.nbref_backward.restype = ctypes.c_int
    ins = [np.ascontiguousarray(a, dtype=np.float32).copy() for a in inputs]
    n_in = len(ins)
    accum = [False] * n_in if accum is None else list(accum)
    if in_grads is None:
        in_grads = [None] * n_in
    grads = [np.zeros_like(a) if g is None else np.ascontiguousarray(g, dtype=np.float32).copy().reshape(a.shape)
             for a, g in zip(ins, in_grads)]
    s = (ctypes.c_double * max(1, len(scalars)))(*[float(v) for v in scalars])
    flat = [int(v) for vec in ivecs for v in vec]
    iv = (ctypes.c_int32 * max(1, len(flat)))(*flat)
    ivl = (ctypes.c_int32 * max(1, len(ivecs)))(*[len(v) for v in ivecs])

    def tensors(arrays):
        t = (_Tensor * len(arrays))()
        for e, a in zip(t, arrays):
            e.data = a.ctypes.data
            e.ndim = a.ndim
            for d, n in enumerate(a.shape):
                e.shape[d] = n
        return t
    n_out = len(out_grads)
    ogs = [np.ascontiguousarray(g, dtype=np.float32).copy() for g in out_grads]
    outs = [np.empty(g.shape, dtype=np.float32) for g in ogs]
    tin, tgin, tout, tgout = tensors(ins), tensors(grads), tensors(outs), tensors(ogs)
    pd = (ctypes.c_int32 * n_in)(*[int(bool(v)) for v in propagate_down])
    ac = (ctypes.c_int32 * n_in)(*[int(bool(v)) for v in accum])
    rc = L.nbref_backward(op.encode(), s, len(scalars), iv, ivl, len(ivecs), tin, tgin, n_in, tout, tgout, n_out,
                          pd, ac)
    if rc != 0:
        raise RuntimeError(L.nbref_last_error().decode())
    for t, o in zip(tout, outs):
        if tuple(t.shape[d] for d in range(t.ndim)) != o.shape:
            raise RuntimeError("out_grads[.] does not have the output's shape")
    return grads, outs, ins


# Convenience wrappers named after the reference functions -------------------

def fixed_point_quantize(x, sign=True, n=8, delta=2.0 ** -4, ste_fine_grained=True, repeat=1, timed=False):
    o, _, t = forward("FixedPointQuantize", [sign, n, delta, ste_fine_grained], [], [x], repeat=repeat)
    return (o[0], t) if timed else o[0]


def pow2_quantize(x, sign=True, with_zero=True, n=8, m=1, ste_fine_grained=True, repeat=1, timed=False):
    o, _, t = forward("Pow2Quantize", [sign, with_zero, n, m, ste_fine_grained], [], [x], repeat=repeat)
    return (o[0], t) if timed else o[0]


def min_max_quantize(x, qr_min, qr_max, ql_min, ql_max, decay=0.999, x_min_max=False, ema=False,
                     ste_fine_grained=True, eps=0.01, repeat=1, timed=False):
    """Returns (y, qr_min_after, qr_max_after[, seconds])."""
    o, i, t = forward("MinMaxQuantize", [decay, x_min_max, ema, ste_fine_grained, eps], [],
                      [x, qr_min, qr_max, ql_min, ql_max], repeat=repeat)
    r = (o[0], i[1], i[2])
    return r + (t,) if timed else r


def sign(x, alpha=1.0):
    return forward("Sign", [alpha], [], [x])[0][0]


def binary_weight_affine(x, w, b=None, base_axis=1, quantize_zero_to=1.0, repeat=1, timed=False):
    """Returns (y, wb, alpha[, seconds])."""
    wb = np.zeros_like(w, dtype=np.float32)
    alpha = np.zeros(int(np.prod(w.shape[1:])), dtype=np.float32)
    o, i, t = forward("BinaryWeightAffine", [base_axis, quantize_zero_to], [], [x, w, wb, alpha, b], repeat=repeat)
    r = (o[0], i[2], i[3])
    return r + (t,) if timed else r


def binary_connect_affine(x, w, b=None, base_axis=1, quantize_zero_to=1.0):
    wb = np.zeros_like(w, dtype=np.float32)
    o, i, _ = forward("BinaryConnectAffine", [base_axis, quantize_zero_to], [], [x, w, wb, b])
    return o[0], i[2]


def binary_weight_convolution(x, w, b=None, base_axis=1, pad=(0, 0), stride=(1, 1), dilation=(1, 1), group=1,
                              quantize_zero_to=1.0, repeat=1, timed=False):
    wb = np.zeros_like(w, dtype=np.float32)
    alpha = np.zeros(w.shape[0], dtype=np.float32)
    o, i, t = forward("BinaryWeightConvolution", [base_axis, group, quantize_zero_to], [pad, stride, dilation],
                      [x, w, wb, alpha, b], repeat=repeat)
    r = (o[0], i[2], i[3])
    return r + (t,) if timed else r


def binary_connect_convolution(x, w, b=None, base_axis=1, pad=(0, 0), stride=(1, 1), dilation=(1, 1), group=1,
                               quantize_zero_to=1.0):
    wb = np.zeros_like(w, dtype=np.float32)
    o, i, _ = forward("BinaryConnectConvolution", [base_axis, group, quantize_zero_to], [pad, stride, dilation],
                      [x, w, wb, b])
    return o[0], i[2]


def affine(x, w, b=None, base_axis=1, repeat=1, timed=False):
    o, _, t = forward("Affine", [base_axis], [], [x, w, b], repeat=repeat)
    return (o[0], t) if timed else o[0]


def convolution(x, w, b=None, base_axis=1, pad=(0, 0), stride=(1, 1), dilation=(1, 1), group=1, repeat=1, timed=False):
    o, _, t = forward("Convolution", [base_axis, group, False], [pad, stride, dilation], [x, w, b], repeat=repeat)
    return (o[0], t) if timed else o[0]


def batch_normalization(x, beta, gamma, mean, var, axes=(1,), decay_rate=0.9, eps=1e-5, batch_stat=False):
    o, _, _ = forward("BatchNormalization", [decay_rate, eps, batch_stat, False, False], [axes],
                      [x, beta, gamma, mean, var])
    return o[0]


def relu(x):
    return forward("ReLU", [False], [], [x])[0][0]


def add2(a, b):
    return forward("Add2", [False], [], [a, b])[0][0]


def max_pooling(x, kernel, stride, ignore_border=True, pad=(0, 0)):
    return forward("MaxPooling", [ignore_border, False], [kernel, stride, pad], [x])[0][0]


def average_pooling(x, kernel, stride, ignore_border=True, pad=(0, 0), including_pad=True):
    return forward("AveragePooling", [ignore_border, False, including_pad], [kernel, stride, pad], [x])[0][0]


def global_average_pooling(x):
    return forward("GlobalAveragePooling", [], [], [x])[0][0]


# Backward passes -------------------------------------------------------------

def fixed_point_quantize_backward(x, dy, sign=True, n=8, delta=2.0 ** -4, ste_fine_grained=True, accum=False, dx=None):
    g, _, _ = backward("FixedPointQuantize", [sign, n, delta, ste_fine_grained], [], [x], [dy], [True], [accum], [dx])
    return g[0]


def pow2_quantize_backward(x, dy, sign=True, with_zero=True, n=8, m=1, ste_fine_grained=True, accum=False, dx=None):
    g, _, _ = backward("Pow2Quantize", [sign, with_zero, n, m, ste_fine_grained], [], [x], [dy], [True], [accum], [dx])
    return g[0]


def min_max_quantize_backward(x, qr_min, qr_max, ql_min, ql_max, dy, decay=0.999, x_min_max=False, ema=False,
                              ste_fine_grained=True, eps=0.01, propagate_down=(True, True, True),
                              accum=(False, False, False), grads=(None, None, None)):
    """Returns (dx, g_qr_min, g_qr_max) after forward + backward."""
    pd = list(propagate_down) + [False, False]
    ac = list(accum) + [False, False]
    g, _, _ = backward("MinMaxQuantize", [decay, x_min_max, ema, ste_fine_grained, eps], [],
                       [x, qr_min, qr_max, ql_min, ql_max], [dy], pd, ac, list(grads) + [None, None])
    return g[0], g[1], g[2]


def affine_backward(x, w, b, dy, base_axis=1, propagate_down=(True, True, True), accum=(False, False, False),
                    grads=(None, None, None)):
    """Returns (dx, dw, db) from Affine::backward (b may be None)."""
    ins = [x, w] + ([b] if b is not None else [])
    n = len(ins)
    g, _, _ = backward("Affine", [base_axis], [], ins, [dy], list(propagate_down)[:n], list(accum)[:n],
                       list(grads)[:n])
    return tuple(g) + (None,) * (3 - n)


def binary_weight_affine_backward(x, w, b, dy, base_axis=1, quantize_zero_to=1.0, propagate_down=(True, True, True),
                                  accum=(False, False, False), grads=(None, None, None)):
    """Returns (dx, dw, db) from BinaryWeightAffine::backward; inputs are [x, w, wb, alpha, b?]."""
    wb = np.zeros_like(w, dtype=np.float32)
    alpha = np.zeros(int(np.prod(w.shape[1:])), dtype=np.float32)
    ins = [x, w, wb, alpha] + ([b] if b is not None else [])
    pd = [propagate_down[0], propagate_down[1], False, False] + ([propagate_down[2]] if b is not None else [])
    ac = [accum[0], accum[1], False, False] + ([accum[2]] if b is not None else [])
    g0 = [grads[0], grads[1], None, None] + ([grads[2]] if b is not None else [])
    g, _, _ = backward("BinaryWeightAffine", [base_axis, quantize_zero_to], [], ins, [dy], pd, ac, g0)
    return g[0], g[1], (g[4] if b is not None else None)


def binary_connect_affine_backward(x, w, b, dy, base_axis=1, quantize_zero_to=1.0, propagate_down=(True, True, True),
                                   accum=(False, False, False), grads=(None, None, None)):
    """Returns (dx, dw, db) from BinaryConnectAffine::backward; inputs are [x, w, wb, b?]."""
    wb = np.zeros_like(w, dtype=np.float32)
    ins = [x, w, wb] + ([b] if b is not None else [])
    pd = [propagate_down[0], propagate_down[1], False] + ([propagate_down[2]] if b is not None else [])
    ac = [accum[0], accum[1], False] + ([accum[2]] if b is not None else [])
    g0 = [grads[0], grads[1], None] + ([grads[2]] if b is not None else [])
    g, _, _ = backward("BinaryConnectAffine", [base_axis, quantize_zero_to], [], ins, [dy], pd, ac, g0)
    return g[0], g[1], (g[3] if b is not None else None)


def _conv_backward(op, scalars, ivecs, x, w, extra, b, dy, propagate_down, accum, grads):
    ins = [x, w] + extra + ([b] if b is not None else [])
    ne = len(extra)
    pd = [propagate_down[0], propagate_down[1]] + [False] * ne + ([propagate_down[2]] if b is not None else [])
    ac = [accum[0], accum[1]] + [False] * ne + ([accum[2]] if b is not None else [])
    g0 = [grads[0], grads[1]] + [None] * ne + ([grads[2]] if b is not None else [])
    g, _, _ = backward(op, scalars, ivecs, ins, [dy], pd, ac, g0)
    return g[0], g[1], (g[2 + ne] if b is not None else None)


def convolution_backward(x, w, b, dy, base_axis=1, pad=(0, 0), stride=(1, 1), dilation=(1, 1), group=1,
                         propagate_down=(True, True, True), accum=(False, False, False), grads=(None, None, None)):
    """Returns (dx, dw, db) from Convolution::backward."""
    return _conv_backward("Convolution", [base_axis, group, False], [pad, stride, dilation], x, w, [], b, dy,
                          propagate_down, accum, grads)


def binary_weight_convolution_backward(x, w, b, dy, base_axis=1, pad=(0, 0), stride=(1, 1), dilation=(1, 1), group=1,
                                       quantize_zero_to=1.0, propagate_down=(True, True, True),
                                       accum=(False, False, False), grads=(None, None, None)):
    wb = np.zeros_like(w, dtype=np.float32)
    alpha = np.zeros(w.shape[0], dtype=np.float32)
    return _conv_backward("BinaryWeightConvolution", [base_axis, group, quantize_zero_to], [pad, stride, dilation], x,
                          w, [wb, alpha], b, dy, propagate_down, accum, grads)


def binary_connect_convolution_backward(x, w, b, dy, base_axis=1, pad=(0, 0), stride=(1, 1), dilation=(1, 1),
                                        group=1, quantize_zero_to=1.0, propagate_down=(True, True, True),
                                        accum=(False, False, False), grads=(None, None, None)):
    wb = np.zeros_like(w, dtype=np.float32)
    return _conv_backward("BinaryConnectConvolution", [base_axis, group, quantize_zero_to], [pad, stride, dilation],
                          x, w, [wb], b, dy, propagate_down, accum, grads)


# Sibling quantization functions -------------------------------------------------

def batch_normalization_batch(x, beta, gamma, mean, var, axes=(1,), decay_rate=0.9, eps=1e-5):
    """Batch-statistics forward. Returns (y, batch mean, batch var, running mean after, running var after)."""
    o, ins, _ = forward("BatchNormalization", [decay_rate, eps, True, False, False], [axes],
                        [x, beta, gamma, mean, var], n_out=3)
    return o[0], o[1], o[2], ins[3], ins[4]


def batch_normalization_backward(x, beta, gamma, mean, var, dy, axes=(1,), decay_rate=0.9, eps=1e-5,
                                 batch_stat=True, dmean=None, dvar=None, propagate_down=(True, True, True),
                                 accum=(False, False, False), grads=(None, None, None)):
    """Returns (dx, dbeta, dgamma) after forward + BatchNormalization::backward."""
    ogs = [dy]
    if batch_stat:
        ogs += [np.zeros_like(mean) if dmean is None else dmean, np.zeros_like(var) if dvar is None else dvar]
    g, _, _ = backward("BatchNormalization", [decay_rate, eps, batch_stat, False, False], [axes],
                       [x, beta, gamma, mean, var], ogs, list(propagate_down) + [False, False],
                       list(accum) + [False, False], list(grads) + [None, None])
    return g[0], g[1], g[2]


def relu_backward(x, dy, accum=False, dx=None):
    return backward("ReLU", [False], [], [x], [dy], [True], [accum], [dx])[0][0]


def add2_backward(a, b, dy, accum=(False, False), grads=(None, None)):
    g, _, _ = backward("Add2", [False], [], [a, b], [dy], [True, True], list(accum), list(grads))
    return g[0], g[1]


def global_average_pooling_backward(x, dy, accum=False, dx=None):
    return backward("GlobalAveragePooling", [], [], [x], [dy], [True], [accum], [dx])[0][0]


def max_pooling_backward(x, dy, kernel, stride, ignore_border=True, pad=(0, 0), accum=False, dx=None):
    return backward("MaxPooling", [ignore_border, False], [kernel, stride, pad], [x], [dy], [True], [accum], [dx])[0][0]


def binary_sigmoid(x):
    return forward("BinarySigmoid", [], [], [x])[0][0]


def binary_tanh(x):
    return forward("BinaryTanh", [], [], [x])[0][0]


def binary_sigmoid_backward(x, dy, accum=False, dx=None):
    return backward("BinarySigmoid", [], [], [x], [dy], [True], [accum], [dx])[0][0]


def binary_tanh_backward(x, dy, accum=False, dx=None):
    return backward("BinaryTanh", [], [], [x], [dy], [True], [accum], [dx])[0][0]


def quantize_linear(x, scale, zero_point, round_mode="HALF_AWAY_FROM_ZERO", narrow_range=False, dtype=1):
    """Returns (y, zero_point_after)."""
    o, i, _ = forward("QuantizeLinear", [round_mode == "HALF_TO_EVEN", narrow_range, dtype], [],
                      [x, scale, zero_point])
    return o[0], i[2]


def dequantize_linear(x, scale, zero_point):
    return forward("DequantizeLinear", [], [], [x, scale, zero_point])[0][0]


def quantize_linear_backward(x, scale, zero_point, dy, round_mode="HALF_AWAY_FROM_ZERO", narrow_range=False, dtype=1,
                             accum=False, dx=None):
    g, _, _ = backward("QuantizeLinear", [round_mode == "HALF_TO_EVEN", narrow_range, dtype], [],
                       [x, scale, zero_point], [dy], [True, False, False], [accum, False, False], [dx, None, None])
    return g[0]


def dequantize_linear_backward(x, scale, zero_point, dy, accum=False, dx=None):
    g, _, _ = backward("DequantizeLinear", [], [], [x, scale, zero_point], [dy], [True, False, False],
                       [accum, False, False], [dx, None, None])
    return g[0]


def prune(x, rate=0.9):
    return forward("Prune", [rate], [], [x])[0][0]
