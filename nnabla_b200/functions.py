"""Host-side mirror of nnabla's function API for the quantized-layer forward path.

Same names, argument order, defaults and error behaviour as
python/src/nnabla/functions.py:416-692 (quantizers) and the generated
function_bases for the binary layers, so code and tests written against
`nnabla.functions` read the same here. Arrays are torch CUDA tensors (torch
only provides device memory and streams); every computation is one call into
libnnabla_b200.so. There is no CPU path.
"""
import ctypes
import weakref

import torch

from . import _capi as C


def _check_input(x, name="x"):
    if not isinstance(x, torch.Tensor):
        raise TypeError("%s must be a torch.Tensor on a CUDA device" % name)
    if not x.is_cuda:
        raise RuntimeError("nnabla_b200 has no CPU path: %s is on %s" % (name, x.device))
    if x.dtype != torch.float32:
        raise TypeError("%s must be float32 (the 'float' type config), got %s" % (name, x.dtype))
    return x if x.is_contiguous() else x.contiguous()


def _output_like(x, outputs):
    if outputs is None:
        return torch.empty_like(x)
    y = outputs[0] if isinstance(outputs, (list, tuple)) else outputs
    _sideband.pop(id(y), None)  # about to be overwritten
    if y.shape != x.shape or y.dtype != x.dtype or y.device != x.device or not y.is_contiguous():
        raise RuntimeError("outputs[0] must be a contiguous tensor of x's shape, dtype and device")
    return y


# int8 channel-last codes that a quantizer left beside its fp32 result: id(result) -> (weak reference to the
# result, its version counter, codes, step). A convolution that is handed the very same tensor object, unmodified,
# reads the codes instead of converting the fp32 values again.
_sideband = {}
# below this many values the extra launch that the convolution then needs for its weights costs more than the
# second pass over the activations that the codes save (measured on a binary-weight ResNet-18: a gain from
# 12.8 M values per tensor upwards, a loss at 6.4 M)
SIDEBAND_MIN_VALUES = 1 << 23


def _sideband_put(y, codes, delta):
    key = id(y)
    _sideband[key] = (weakref.ref(y, lambda _r, key=key: _sideband.pop(key, None)), y._version, codes, float(delta))


def _sideband_get(x, delta):
    e = _sideband.get(id(x))
    if e is None or e[0]() is not x or x._version != e[1] or e[3] != float(delta):
        return None
    return e[2]


def fixed_point_quantize(x, sign=True, n=8, delta=2 ** -4, quantize=True, ste_fine_grained=True, outputs=None,
                         codes_sideband=False):
    """Fixed Point Quantize (python/src/nnabla/functions.py:416-482).

    Forward of FixedPointQuantize (src/nbla/function/generic/fixed_point_quantize.cpp:45-66).
    codes_sideband=True (an [N, C, H, W] tensor of at least SIDEBAND_MIN_VALUES values with H * W a multiple of 4,
    n - sign <= 7; otherwise the plain quantizer runs): the same pass also
    writes the result's int8 channel-last codes and keeps them with the returned tensor; a binary-weight
    convolution called on that tensor with fixed_point_delta=delta then reads the codes. The result is the
    same, bit for bit. The codes are dropped when the tensor is modified through torch or passed as `outputs`
    of a function of this module; do not write into it any other way.
    """
    if not quantize:
        return x
    x = _check_input(x)
    y = _output_like(x, outputs)
    if (codes_sideband and x.dim() == 4 and (int(x.shape[2]) * int(x.shape[3])) % 4 == 0
            and x.numel() >= SIDEBAND_MIN_VALUES
            and int(n) - int(bool(sign)) <= 7 and int(x.shape[0]) <= 65535 and x.data_ptr() % 16 == 0
            and y.data_ptr() % 16 == 0):
        N, Cn, inner = int(x.shape[0]), int(x.shape[1]), int(x.shape[2]) * int(x.shape[3])
        codes = torch.empty((N, inner, codes_nhwc_slots(Cn, 1)), dtype=torch.int8, device=x.device)
        with C.on_device(x.device):
            C.call("nb200_fixed_point_quantize_nhwc_codes_f32", C.ptr(x), C.ptr(y), C.ptr(codes), N, Cn, inner,
                   int(bool(sign)), int(n), C.c_float(delta), C.stream_ptr(x.device))
        _sideband_put(y, codes, delta)
        return y
    with C.on_device(x.device):
        C.call("nb200_fixed_point_quantize_f32", C.ptr(x), C.ptr(y), C.size_t(x.numel()), int(bool(sign)), int(n),
               C.c_float(delta), C.stream_ptr(x.device))
    return y


def fixed_point_quantize_with_codes(x, sign=True, n=8, delta=2 ** -4):
    """fixed_point_quantize that also returns the int8 codes k (y = k * delta)."""
    x = _check_input(x)
    y = torch.empty_like(x)
    codes = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    with C.on_device(x.device):
        C.call("nb200_fixed_point_quantize_f32_codes", C.ptr(x), C.ptr(y), C.ptr(codes), C.size_t(x.numel()),
               int(bool(sign)), int(n), C.c_float(delta), C.stream_ptr(x.device))
    return y, codes


def pow2_quantize(x, sign=True, with_zero=True, n=8, m=1, quantize=True, ste_fine_grained=True, outputs=None):
    """Pow2 Quantize (python/src/nnabla/functions.py:485-580).

    Forward of Pow2Quantize (src/nbla/function/generic/pow2_quantize.cpp:47-82).
    """
    if not quantize:
        return x
    x = _check_input(x)
    y = _output_like(x, outputs)
    with C.on_device(x.device):
        C.call("nb200_pow2_quantize_f32", C.ptr(x), C.ptr(y), C.size_t(x.numel()), int(bool(sign)),
               int(bool(with_zero)), int(n), int(m), C.stream_ptr(x.device))
    return y


def min_max_quantize(x, qr_min, qr_max, ql_min, ql_max, decay=0.999, x_min_max=False, ema=False,
                     ste_fine_grained=True, eps=0.01, quantize=True, outputs=None):
    """Min-max quantization (python/src/nnabla/functions.py:583-692).

    Forward of MinMaxQuantize (src/nbla/function/generic/min_max_quantize.cpp:129-223).
    As in the reference, qr_min and qr_max are UPDATED IN PLACE (min/max of x
    or their moving average when x_min_max; the eps nudge of qr_max always).
    """
    if not quantize:
        return x
    x = _check_input(x)
    qs = [_check_input(t, nm) for t, nm in ((qr_min, "qr_min"), (qr_max, "qr_max"), (ql_min, "ql_min"),
                                            (ql_max, "ql_max"))]
    # Shape rules of MinMaxQuantize::setup_impl (min_max_quantize.cpp:54-83).
    if len({t.dim() for t in qs}) != 1:
        raise RuntimeError("All input dimensions must be same.")
    if len({tuple(t.shape) for t in qs}) != 1:
        raise RuntimeError("All shapes among ql_min, ql_max, qr_min, and qr_max must be same.")
    if qs[0].dim() != x.dim():
        raise RuntimeError("x.shape and ql_min.shape must be same except for i-th dimension where "
                           "ql_min.shape[i] == 1.")
    for t, orig in zip(qs[:2], (qr_min, qr_max)):
        if t is not orig:
            raise RuntimeError("qr_min and qr_max are updated in place and must be contiguous")
    y = _output_like(x, outputs)
    with C.on_device(x.device):
        C.call("nb200_min_max_quantize_f32", C.ptr(x), C.i64_array(x.shape), int(x.dim()), C.ptr(qs[0]),
               C.ptr(qs[1]), C.ptr(qs[2]), C.ptr(qs[3]), C.i64_array(qs[0].shape), C.c_float(decay),
               int(bool(x_min_max)), int(bool(ema)), C.c_float(eps), C.ptr(y), ctypes.c_void_p(0),
               C.stream_ptr(x.device))
    return y


# ---------------------------------------------------------------------------
# Quantizer backward passes. nnabla reaches these through Function::backward of
# the graph engine; here they are plain calls: dx receives (accum=False) or
# accumulates (accum=True) the gradient w.r.t. x given the output gradient dy.
# ---------------------------------------------------------------------------

def _grad_buffers(x, dy, dx, accum):
    x, dy = _check_input(x), _check_input(dy, "dy")
    if dy.shape != x.shape:
        raise RuntimeError("dy must have x's shape")
    if dx is None:
        if accum:
            raise RuntimeError("accum=True needs the gradient buffer dx to accumulate into")
        dx = torch.empty_like(x)
    elif dx.shape != x.shape or dx.dtype != torch.float32 or dx.device != x.device or not dx.is_contiguous():
        raise RuntimeError("dx must be a contiguous float32 tensor of x's shape and device")
    return x, dy, dx


def fixed_point_quantize_backward(x, dy, sign=True, n=8, delta=2 ** -4, ste_fine_grained=True, accum=False, dx=None):
    """FixedPointQuantize::backward_impl (src/nbla/function/generic/fixed_point_quantize.cpp:69-127)."""
    x, dy, dx = _grad_buffers(x, dy, dx, accum)
    with C.on_device(x.device):
        C.call("nb200_fixed_point_quantize_backward_f32", C.ptr(x), C.ptr(dy), C.ptr(dx), C.size_t(x.numel()),
               int(bool(sign)), int(n), C.c_float(delta), int(bool(ste_fine_grained)), int(bool(accum)),
               C.stream_ptr(x.device))
    return dx


def pow2_quantize_backward(x, dy, sign=True, with_zero=True, n=8, m=1, ste_fine_grained=True, accum=False, dx=None):
    """Pow2Quantize::backward_impl (src/nbla/function/generic/pow2_quantize.cpp:84-156)."""
    x, dy, dx = _grad_buffers(x, dy, dx, accum)
    with C.on_device(x.device):
        C.call("nb200_pow2_quantize_backward_f32", C.ptr(x), C.ptr(dy), C.ptr(dx), C.size_t(x.numel()),
               int(bool(sign)), int(bool(with_zero)), int(n), int(m), int(bool(ste_fine_grained)), int(bool(accum)),
               C.stream_ptr(x.device))
    return dx


def min_max_quantize_backward(x, qr_min, qr_max, ql_min, ql_max, dy, x_min_max=False, ema=False,
                              ste_fine_grained=True, propagate_down=(True, True, True),
                              accum=(False, False, False), grads=(None, None, None)):
    """MinMaxQuantize::backward_impl (src/nbla/function/generic/min_max_quantize.cpp:225-350).

    Call after min_max_quantize: qr_min / qr_max are the ranges the forward
    left in place. Returns (dx, g_qr_min, g_qr_max); the range gradients are
    produced only when neither x_min_max nor ema is set."""
    x, dy, dx = _grad_buffers(x, dy, grads[0], accum[0])
    qs = [_check_input(t, nm) for t, nm in ((qr_min, "qr_min"), (qr_max, "qr_max"), (ql_min, "ql_min"),
                                            (ql_max, "ql_max"))]
    if len({tuple(t.shape) for t in qs}) != 1 or qs[0].dim() != x.dim():
        raise RuntimeError("All shapes among ql_min, ql_max, qr_min, and qr_max must be same.")
    gq = []
    for g, acc in ((grads[1], accum[1]), (grads[2], accum[2])):
        if g is None:
            if acc:
                raise RuntimeError("accum=True needs the gradient buffer to accumulate into")
            g = torch.zeros_like(qs[0])
        gq.append(_check_input(g, "range gradient"))
    with C.on_device(x.device):
        C.call("nb200_min_max_quantize_backward_f32", C.ptr(x), C.i64_array(x.shape), int(x.dim()), C.ptr(qs[0]),
               C.ptr(qs[1]), C.ptr(qs[2]), C.ptr(qs[3]), C.i64_array(qs[0].shape), C.ptr(dy), int(bool(x_min_max)),
               int(bool(ema)), int(bool(ste_fine_grained)), C.i32_array([bool(v) for v in propagate_down]),
               C.i32_array([bool(v) for v in accum]), C.ptr(dx), C.ptr(gq[0]), C.ptr(gq[1]),
               C.stream_ptr(x.device))
    return dx, gq[0], gq[1]


# ---------------------------------------------------------------------------
# Affine layers
# ---------------------------------------------------------------------------

def check_device_status(device=None):
    """Raises if a bounded device-side wait gave up since the last check
    (synchronises the current stream)."""
    code = ctypes.c_int(0)
    C.call("nb200_take_device_status", ctypes.byref(code), C.stream_ptr(device))
    if code.value != 0:
        raise C.NB200Error(5, "a device-side wait gave up (status 0x%x); results are incomplete" % code.value)


def _affine_dims(x, w, base_axis, bias):
    """Shape rules of Affine::setup_impl (src/nbla/function/generic/affine.cpp:29-78)."""
    if w.dim() < 2:
        raise RuntimeError("Weights(inputs[1]) must be matrix or tensor.")
    if base_axis < 0:
        base_axis += x.dim()
    if not 0 <= base_axis < x.dim():
        raise RuntimeError("Base_axis must be less than ndim of input data(inputs[0]). base_axis: %d >= ndim of "
                           "input: %d." % (base_axis, x.dim()))
    rows = 1
    for s in x.shape[:base_axis]:
        rows *= int(s)
    i_col = x.numel() // max(rows, 1)
    w_row = int(w.shape[0])
    w_col = w.numel() // max(w_row, 1)
    if i_col != w_row:
        raise RuntimeError("Size of input data(inputs[0]) and weights(inputs[1]) mismatch. size of input: %d != "
                           "size of weights: %d." % (i_col, w_row))
    if bias is not None:
        if bias.dim() != w.dim() - 1 or tuple(bias.shape) != tuple(w.shape[1:]):
            raise RuntimeError("Shape of bias(inputs[2]) and weights(inputs[1]) mismatch.")
    out_shape = tuple(x.shape[:base_axis]) + tuple(w.shape[1:])
    return rows, w_row, w_col, out_shape


def _same_shape(a, b, what):
    if a.dim() != b.dim() or tuple(a.shape) != tuple(b.shape):
        raise RuntimeError("Binary and float weights must have same size. (%s)" % what)


def binary_weight_affine(x, weight, binary_weight, alpha, bias=None, base_axis=1, quantize_zero_to=1.0,
                         n_outputs=-1, outputs=None):
    """Binary Weight Affine (function_bases.binary_weight_affine).

    Forward of BinaryWeightAffine (src/nbla/function/generic/binary_weight_affine.cpp:74-122):
    writes `binary_weight` = sign(weight) and `alpha` = mean |weight| per output,
    returns x . binary_weight * alpha + bias.
    """
    x, weight = _check_input(x), _check_input(weight, "weight")
    binary_weight, alpha = _check_input(binary_weight, "binary_weight"), _check_input(alpha, "alpha")
    bias = _check_input(bias, "bias") if bias is not None else None
    rows, w_row, w_col, out_shape = _affine_dims(x, weight, base_axis, bias)
    _same_shape(weight, binary_weight, "float vs binary")
    if alpha.numel() != w_col:
        raise RuntimeError("Size of alpha must be equal to output size.")
    y = torch.empty(out_shape, dtype=torch.float32, device=x.device) if outputs is None else outputs[0]
    with C.on_device(x.device):
        C.call("nb200_binary_weight_affine_f32", C.ptr(x), C.ptr(weight), C.ptr(binary_weight), C.ptr(alpha),
               C.ptr(bias), C.ptr(y), ctypes.c_int64(rows), ctypes.c_int64(w_row), ctypes.c_int64(w_col),
               C.c_float(quantize_zero_to), C.stream_ptr(x.device))
    return y


def binary_connect_affine(x, weight, binary_weight, bias=None, base_axis=1, quantize_zero_to=1.0, n_outputs=-1,
                          outputs=None):
    """Binary Connect Affine (function_bases.binary_connect_affine).

    Forward of BinaryConnectAffine (src/nbla/function/generic/binary_connect_affine.cpp:59-71).
    """
    x, weight = _check_input(x), _check_input(weight, "weight")
    binary_weight = _check_input(binary_weight, "binary_weight")
    bias = _check_input(bias, "bias") if bias is not None else None
    rows, w_row, w_col, out_shape = _affine_dims(x, weight, base_axis, bias)
    _same_shape(weight, binary_weight, "float vs binary")
    y = torch.empty(out_shape, dtype=torch.float32, device=x.device) if outputs is None else outputs[0]
    with C.on_device(x.device):
        C.call("nb200_binary_connect_affine_f32", C.ptr(x), C.ptr(weight), C.ptr(binary_weight), C.ptr(bias),
               C.ptr(y), ctypes.c_int64(rows), ctypes.c_int64(w_row), ctypes.c_int64(w_col),
               C.c_float(quantize_zero_to), C.stream_ptr(x.device))
    return y


def affine(x, weight, bias=None, base_axis=1, n_outputs=-1, outputs=None, fixed_point=None):
    """Affine (function_bases.affine; src/nbla/function/generic/affine.cpp:80-96).

    fixed_point=(delta_x, delta_w): x and weight are outputs of
    fixed_point_quantize with n <= 8 and those step sizes; the product then
    runs on the int8 tensor-core path. Otherwise the fp32-accurate split path.
    """
    x, weight = _check_input(x), _check_input(weight, "weight")
    bias = _check_input(bias, "bias") if bias is not None else None
    rows, w_row, w_col, out_shape = _affine_dims(x, weight, base_axis, bias)
    y = torch.empty(out_shape, dtype=torch.float32, device=x.device) if outputs is None else outputs[0]
    with C.on_device(x.device):
        if fixed_point is not None:
            dx, dw = fixed_point
            C.call("nb200_affine_fxp8_f32", C.ptr(x), C.ptr(weight), C.c_float(dx), C.c_float(dw), C.ptr(bias),
                   C.ptr(y), ctypes.c_int64(rows), ctypes.c_int64(w_row), ctypes.c_int64(w_col),
                   C.stream_ptr(x.device))
        else:
            C.call("nb200_affine_f32", C.ptr(x), C.ptr(weight), C.ptr(bias), C.ptr(y), ctypes.c_int64(rows),
                   ctypes.c_int64(w_row), ctypes.c_int64(w_col), C.stream_ptr(x.device))
    return y


def affine_from_codes(x_codes, w_codes, delta_x, delta_w, bias=None):
    """Affine on the int8 codes written by fixed_point_quantize_with_codes
    (x_codes [rows, K], w_codes [K, N])."""
    rows, K = x_codes.shape
    K2, N = w_codes.shape
    if K != K2:
        raise RuntimeError("Size of input data(inputs[0]) and weights(inputs[1]) mismatch.")
    y = torch.empty((rows, N), dtype=torch.float32, device=x_codes.device)
    with C.on_device(x_codes.device):
        C.call("nb200_affine_codes_i8_f32", C.ptr(x_codes), C.ptr(w_codes), C.c_float(delta_x), C.c_float(delta_w),
               C.ptr(bias), C.ptr(y), ctypes.c_int64(rows), ctypes.c_int64(K), ctypes.c_int64(N),
               C.stream_ptr(x_codes.device))
    return y


def _affine_backward(entry, x, w, alpha, dy, base_axis, propagate_down, accum, grads):
    """Shared driver of the affine backward entry points. Returns (dx, dw, db);
    an entry whose propagate_down flag is false is returned as passed in."""
    x, w, dy = _check_input(x), _check_input(w, "weight"), _check_input(dy, "dy")
    rows, w_row, w_col, out_shape = _affine_dims(x, w, base_axis, None)
    if tuple(dy.shape) != tuple(out_shape):
        raise RuntimeError("dy must have the output's shape")
    shapes = (x.shape, w.shape, w.shape[1:])
    out = []
    for g, shape, pd, ac in zip(grads, shapes, propagate_down, accum):
        if not pd:
            out.append(g)
            continue
        if g is None:
            if ac:
                raise RuntimeError("accum=True needs the gradient buffer to accumulate into")
            g = torch.empty(tuple(shape), dtype=torch.float32, device=x.device)
        elif tuple(g.shape) != tuple(shape) or g.dtype != torch.float32 or not g.is_cuda or not g.is_contiguous():
            raise RuntimeError("gradient buffers must be contiguous float32 CUDA tensors of their input's shape")
        out.append(g)
    p = [C.ptr(g) if pd else ctypes.c_void_p(0) for g, pd in zip(out, propagate_down)]
    args = [C.ptr(x), C.ptr(w)] + ([C.ptr(alpha)] if alpha is not None else []) + [C.ptr(dy)] + p + [
        ctypes.c_int64(rows), ctypes.c_int64(w_row), ctypes.c_int64(w_col), int(bool(accum[0])), int(bool(accum[1])),
        int(bool(accum[2])), C.stream_ptr(x.device)]
    with C.on_device(x.device):
        C.call(entry, *args)
    return tuple(out)


def affine_backward(x, weight, dy, base_axis=1, propagate_down=(True, True, True), accum=(False, False, False),
                    grads=(None, None, None)):
    """Affine::backward_impl (src/nbla/function/generic/affine.cpp:98-138): returns (dx, dw, db)."""
    return _affine_backward("nb200_affine_backward_f32", x, weight, None, dy, base_axis, propagate_down, accum, grads)


def binary_weight_affine_backward(x, binary_weight, alpha, dy, base_axis=1, propagate_down=(True, True, True),
                                  accum=(False, False, False), grads=(None, None, None)):
    """BinaryWeightAffine::backward_impl (src/nbla/function/generic/binary_weight_affine.cpp:124-146).

    binary_weight / alpha are what the forward wrote; dw is the gradient of the
    FLOAT weights (the gradient of the scaled binary weights passes straight
    through Sign). Returns (dx, dw, db)."""
    alpha = _check_input(alpha, "alpha")
    return _affine_backward("nb200_binary_weight_affine_backward_f32", x, binary_weight, alpha, dy, base_axis,
                            propagate_down, accum, grads)


def binary_connect_affine_backward(x, binary_weight, dy, base_axis=1, propagate_down=(True, True, True),
                                   accum=(False, False, False), grads=(None, None, None)):
    """BinaryConnectAffine::backward_impl (src/nbla/function/generic/binary_connect_affine.cpp:73-93)."""
    return _affine_backward("nb200_binary_connect_affine_backward_f32", x, binary_weight, None, dy, base_axis,
                            propagate_down, accum, grads)


def transpose_codes(w_codes):
    """K-major copy [N][Kp] (Kp = K rounded up to 16, zero padded) of int8 weight
    codes [K, N]: the layout affine_from_codes(..., w_kmajor=True) reads without
    a re-layout pass. Done once per weight update."""
    K, N = w_codes.shape
    Kp = (K + 15) // 16 * 16
    out = torch.empty((N, Kp), dtype=torch.int8, device=w_codes.device)
    with C.on_device(w_codes.device):
        C.call("nb200_transpose_codes_i8", C.ptr(w_codes.contiguous()), C.ptr(out), ctypes.c_int64(K),
               ctypes.c_int64(N), ctypes.c_int64(Kp), C.stream_ptr(w_codes.device))
    return out


def affine_from_kmajor_codes(x_codes, w_codes_kmajor, w_row, delta_x, delta_w, bias=None):
    """affine_from_codes with weight codes prepared by transpose_codes ([N][Kp])."""
    rows, K = x_codes.shape
    N, Kp = w_codes_kmajor.shape
    if K != w_row or Kp < K:
        raise RuntimeError("Size of input data(inputs[0]) and weights(inputs[1]) mismatch.")
    y = torch.empty((rows, N), dtype=torch.float32, device=x_codes.device)
    with C.on_device(x_codes.device):
        C.call("nb200_affine_codes_i8_kmajor_f32", C.ptr(x_codes), C.ptr(w_codes_kmajor), ctypes.c_int64(Kp),
               C.c_float(delta_x), C.c_float(delta_w), C.ptr(bias), C.ptr(y), ctypes.c_int64(rows), ctypes.c_int64(K),
               ctypes.c_int64(N), C.stream_ptr(x_codes.device))
    return y


def _rank_pointers(y_ranks):
    """ctypes array of the per-rank output matrices' device addresses (tensors or plain integers)."""
    addrs = [int(y.data_ptr()) if hasattr(y, "data_ptr") else int(y) for y in y_ranks]
    return (ctypes.c_void_p * len(addrs))(*addrs)


def affine_from_codes_gather(x_codes, w_codes, delta_x, delta_w, bias, y_ranks, rank, n_total, col_begin):
    """Column shard of affine_from_codes with the gather fused into the kernel.

    w_codes [K, n] and bias [n] are this rank's slab, columns [col_begin,
    col_begin + n) of a [K, n_total] weight. y_ranks lists, for every rank, the
    device address (or tensor) of its row-major [rows, n_total] fp32 result as
    seen from this process (sharding.PeerMatrices provides them); the slab is
    stored into all of them. The full result is valid on a rank once every
    rank's call has completed (PeerMatrices.fence)."""
    rows, K = x_codes.shape
    K2, n = w_codes.shape
    if K != K2:
        raise RuntimeError("Size of input data(inputs[0]) and weights(inputs[1]) mismatch.")
    with C.on_device(x_codes.device):
        C.call("nb200_affine_codes_i8_gather_f32", C.ptr(x_codes), C.ptr(w_codes), C.c_float(delta_x),
               C.c_float(delta_w), C.ptr(bias), _rank_pointers(y_ranks), int(len(y_ranks)), int(rank),
               ctypes.c_int64(rows), ctypes.c_int64(K), ctypes.c_int64(n), ctypes.c_int64(n_total),
               ctypes.c_int64(col_begin), C.stream_ptr(x_codes.device))


def affine_fixed_point_gather(xq, wq, delta_x, delta_w, bias, y_ranks, rank, n_total, col_begin):
    """As affine_from_codes_gather, from the fp32 outputs of fixed_point_quantize
    (xq [rows, K] multiples of delta_x, wq [K, n] multiples of delta_w)."""
    xq, wq = _check_input(xq, "xq"), _check_input(wq, "wq")
    rows, K = xq.shape
    K2, n = wq.shape
    if K != K2:
        raise RuntimeError("Size of input data(inputs[0]) and weights(inputs[1]) mismatch.")
    with C.on_device(xq.device):
        C.call("nb200_affine_fxp8_gather_f32", C.ptr(xq), C.ptr(wq), C.c_float(delta_x), C.c_float(delta_w),
               C.ptr(bias), _rank_pointers(y_ranks), int(len(y_ranks)), int(rank), ctypes.c_int64(rows),
               ctypes.c_int64(K), ctypes.c_int64(n), ctypes.c_int64(n_total), ctypes.c_int64(col_begin),
               C.stream_ptr(xq.device))


# ---------------------------------------------------------------------------
# Convolutions
# ---------------------------------------------------------------------------

def _conv_geometry(x, w, bias, base_axis, pad, stride, dilation, group):
    """Shape rules of Convolution::setup_impl (src/nbla/function/generic/convolution.cpp:40-158)."""
    if base_axis < 0:
        base_axis += x.dim()
    if not 0 <= base_axis < x.dim() - 1:
        raise RuntimeError("base_axis must be less than ndim - 1 of inputs[0]. base_axis: %d >= ndim of inputs[0] "
                           "- 1: %d." % (base_axis, x.dim() - 1))
    spatial = x.dim() - base_axis - 1
    if w.dim() != 2 + spatial:
        raise RuntimeError("Weights must be a tensor more than 3D.")
    if spatial != 2:
        raise C.NB200Error(4, "only 2-D convolution is implemented (got %d spatial dims)" % spatial)
    pad = (0,) * spatial if pad is None else tuple(pad)
    stride = (1,) * spatial if stride is None else tuple(stride)
    dilation = (1,) * spatial if dilation is None else tuple(dilation)
    for name, v in (("pad", pad), ("stride", stride), ("dilation", dilation)):
        if len(v) != spatial:
            raise RuntimeError("%s size mismatch. %s size: %d != spatial dims: %d." % (name, name, len(v), spatial))
    batch = 1
    for s in x.shape[:base_axis]:
        batch *= int(s)
    Cin, H, W = (int(s) for s in x.shape[base_axis:])
    Ko, Cg, kh, kw = (int(s) for s in w.shape)
    if Cin % group != 0:
        raise RuntimeError("Number of input channel needs to be divisible by group. Input channel: %d, group: %d."
                           % (Cin, group))
    if Ko % group != 0:
        raise RuntimeError("Number of output channel needs to be divisible by group. Output channel: %d, group: %d."
                           % (Ko, group))
    if Cin // group != Cg:
        raise RuntimeError("Number of grouped channel mismatch. Input: %d != Weights[1]: %d." % (Cin // group, Cg))
    if bias is not None and (bias.dim() != 1 or int(bias.shape[0]) != Ko):
        raise RuntimeError("Shape of bias(inputs[2]) and weights(inputs[1]) mismatch.")
    outs = []
    for i, (inp, k) in enumerate(((H, kh), (W, kw))):
        kk = dilation[i] * (k - 1) + 1
        o = (inp + 2 * pad[i] - kk) // stride[i] + 1
        if inp + 2 * pad[i] - kk < 0 or o <= 0:
            raise RuntimeError("Invalid configuration of convolution at %d-th spatial dimension. {input:%d, "
                               "kernel:%d, pad:%d, stride:%d, dilation:%d}." % (i, inp, k, pad[i], stride[i],
                                                                              dilation[i]))
        outs.append(o)
    out_shape = tuple(x.shape[:base_axis]) + (Ko, outs[0], outs[1])
    return batch, Cin, H, W, Ko, kh, kw, pad, stride, dilation, out_shape


def _binary_convolution(entry, x, weight, binary_weight, alpha, bias, base_axis, pad, stride, dilation, group,
                        quantize_zero_to, outputs, fixed_point_delta):
    if fixed_point_delta is not None and group == 1 and base_axis == 1 and x.dim() == 4:
        codes = _sideband_get(x, fixed_point_delta)
        if codes is not None:  # the quantizer that made x left its channel-last codes
            return binary_weight_convolution_from_codes(codes, tuple(x.shape), weight, binary_weight, alpha, bias, pad,
                                                        stride, dilation, group, quantize_zero_to, fixed_point_delta,
                                                        outputs)
    x, weight = _check_input(x), _check_input(weight, "weight")
    binary_weight = _check_input(binary_weight, "binary_weight")
    bias = _check_input(bias, "bias") if bias is not None else None
    batch, Cin, H, W, Ko, kh, kw, pad, stride, dilation, out_shape = _conv_geometry(
        x, weight, bias, base_axis, pad, stride, dilation, group)
    _same_shape(weight, binary_weight, "float vs binary")
    y = torch.empty(out_shape, dtype=torch.float32, device=x.device) if outputs is None else outputs[0]
    args = [C.ptr(x), C.ptr(weight), C.ptr(binary_weight)]
    if alpha is not None:
        args.append(C.ptr(alpha))
    args += [C.ptr(bias), C.ptr(y), batch, Cin, H, W, Ko, kh, kw, pad[0], pad[1], stride[0], stride[1], dilation[0],
             dilation[1], int(group), C.c_float(quantize_zero_to), C.c_float(fixed_point_delta or 0.0),
             C.stream_ptr(x.device)]
    with C.on_device(x.device):
        C.call(entry, *args)
    return y


def binary_weight_convolution(x, weight, binary_weight, alpha, bias=None, base_axis=1, pad=None, stride=None,
                              dilation=None, group=1, quantize_zero_to=1.0, n_outputs=-1, outputs=None,
                              fixed_point_delta=None):
    """Binary Weight Convolution (function_bases.binary_weight_convolution).

    Forward of BinaryWeightConvolution
    (src/nbla/function/generic/binary_weight_convolution.cpp:72-117). Writes
    `binary_weight` and `alpha`. fixed_point_delta=d declares that x is the
    output of fixed_point_quantize with step d and n <= 8, which selects the
    exact int8 contraction.
    """
    alpha = _check_input(alpha, "alpha")
    if alpha.numel() != int(weight.shape[0]):
        raise RuntimeError("Size of alpha must be equal to the number of output maps.")
    return _binary_convolution("nb200_binary_weight_convolution_f32", x, weight, binary_weight, alpha, bias,
                               base_axis, pad, stride, dilation, group, quantize_zero_to, outputs, fixed_point_delta)


def binary_connect_convolution(x, weight, binary_weight, bias=None, base_axis=1, pad=None, stride=None,
                               dilation=None, group=1, quantize_zero_to=1.0, n_outputs=-1, outputs=None,
                               fixed_point_delta=None):
    """Binary Connect Convolution (function_bases.binary_connect_convolution).

    Forward of BinaryConnectConvolution
    (src/nbla/function/generic/binary_connect_convolution.cpp:67-80).
    """
    return _binary_convolution("nb200_binary_connect_convolution_f32", x, weight, binary_weight, None, bias,
                               base_axis, pad, stride, dilation, group, quantize_zero_to, outputs, fixed_point_delta)


def _binary_convolution_backward(entry, x, binary_weight, alpha, dy, base_axis, pad, stride, dilation, group,
                                 propagate_down, accum, grads, fixed_point_delta):
    x, w, dy = _check_input(x), _check_input(binary_weight, "binary_weight"), _check_input(dy, "dy")
    batch, Cin, H, W, Ko, kh, kw, pad, stride, dilation, out_shape = _conv_geometry(
        x, w, None, base_axis, pad, stride, dilation, group)
    if tuple(dy.shape) != tuple(out_shape):
        raise RuntimeError("dy must have the output's shape")
    shapes = (x.shape, w.shape, (Ko,))
    out = []
    for g, shape, pd, ac in zip(grads, shapes, propagate_down, accum):
        if not pd:
            out.append(g)
            continue
        if g is None:
            if ac:
                raise RuntimeError("accum=True needs the gradient buffer to accumulate into")
            g = torch.empty(tuple(shape), dtype=torch.float32, device=x.device)
        elif tuple(g.shape) != tuple(shape) or g.dtype != torch.float32 or not g.is_cuda or not g.is_contiguous():
            raise RuntimeError("gradient buffers must be contiguous float32 CUDA tensors of their input's shape")
        out.append(g)
    p = [C.ptr(g) if pd else ctypes.c_void_p(0) for g, pd in zip(out, propagate_down)]
    args = [C.ptr(x), C.ptr(w)] + ([C.ptr(alpha)] if alpha is not None else []) + [C.ptr(dy)] + p + [
        batch, Cin, H, W, Ko, kh, kw, int(pad[0]), int(pad[1]), int(stride[0]), int(stride[1]), int(dilation[0]),
        int(dilation[1]), int(group), int(bool(accum[0])), int(bool(accum[1])), int(bool(accum[2])),
        C.c_float(fixed_point_delta or 0.0), C.stream_ptr(x.device)]
    with C.on_device(x.device):
        C.call(entry, *args)
    return tuple(out)


def binary_weight_convolution_backward(x, binary_weight, alpha, dy, base_axis=1, pad=None, stride=None, dilation=None,
                                       group=1, propagate_down=(True, True, True), accum=(False, False, False),
                                       grads=(None, None, None), fixed_point_delta=None):
    """BinaryWeightConvolution::backward_impl
    (src/nbla/function/generic/binary_weight_convolution.cpp:119-146): returns
    (dx, dw, db); binary_weight / alpha are what the forward wrote, dw is the
    gradient of the float weights. fixed_point_delta as in the forward."""
    alpha = _check_input(alpha, "alpha")
    return _binary_convolution_backward("nb200_binary_weight_convolution_backward_f32", x, binary_weight, alpha, dy,
                                        base_axis, pad, stride, dilation, group, propagate_down, accum, grads,
                                        fixed_point_delta)


def binary_connect_convolution_backward(x, binary_weight, dy, base_axis=1, pad=None, stride=None, dilation=None,
                                        group=1, propagate_down=(True, True, True), accum=(False, False, False),
                                        grads=(None, None, None), fixed_point_delta=None):
    """BinaryConnectConvolution::backward_impl
    (src/nbla/function/generic/binary_connect_convolution.cpp:82-104)."""
    return _binary_convolution_backward("nb200_binary_connect_convolution_backward_f32", x, binary_weight, None, dy,
                                        base_axis, pad, stride, dilation, group, propagate_down, accum, grads,
                                        fixed_point_delta)


def convolution_backward(x, weight_shape, dy, base_axis=1, pad=None, stride=None, dilation=None, group=1,
                         propagate_down=(False, True, True), accum=(False, False, False), grads=(None, None, None),
                         weight=None):
    """Gradients of the full-precision convolution
    (Convolution::backward_impl, src/nbla/function/generic/convolution.cpp:199-300).
    Returns (dx, dw, db), None where propagate_down is False; dx needs `weight`."""
    x, dy = _check_input(x), _check_input(dy, "dy")
    if weight is not None:
        weight_shape = tuple(_check_input(weight, "weight").shape)
    elif propagate_down[0]:
        raise RuntimeError("the gradient w.r.t. x needs the weights (weight=)")
    w_like = torch.empty(tuple(weight_shape), device="meta")
    batch, Cin, H, W, Ko, kh, kw, pad, stride, dilation, out_shape = _conv_geometry(
        x, w_like, None, base_axis, pad, stride, dilation, group)
    if tuple(dy.shape) != tuple(out_shape):
        raise RuntimeError("dy must have the output's shape")
    out = []
    for g, shape, pd, ac in zip(grads, (tuple(x.shape), tuple(weight_shape), (Ko,)), propagate_down, accum):
        if pd and g is None:
            if ac:
                raise RuntimeError("accum=True needs the gradient buffer to accumulate into")
            g = torch.empty(shape, dtype=torch.float32, device=x.device)
        out.append(g if pd else None)
    with C.on_device(x.device):
        if propagate_down[0]:
            C.call("nb200_convolution_input_backward_f32", C.ptr(weight), C.ptr(dy), C.ptr(out[0]), batch, Cin, H, W, Ko,
                   kh, kw, int(pad[0]), int(pad[1]), int(stride[0]), int(stride[1]), int(dilation[0]),
                   int(dilation[1]), int(group), int(bool(accum[0])), C.stream_ptr(x.device))
        if propagate_down[1] or propagate_down[2]:
            C.call("nb200_convolution_backward_f32", C.ptr(x), C.ptr(dy), C.ptr(out[1]) if propagate_down[1] else
                   ctypes.c_void_p(0), C.ptr(out[2]) if propagate_down[2] else ctypes.c_void_p(0), batch, Cin, H, W, Ko,
                   kh, kw, int(pad[0]), int(pad[1]), int(stride[0]), int(stride[1]), int(dilation[0]),
                   int(dilation[1]), int(group), int(bool(accum[1])), int(bool(accum[2])), C.stream_ptr(x.device))
    return tuple(out)


# ---------------------------------------------------------------------------
# Companion functions of a binary-weight ResNet-18 graph
# ---------------------------------------------------------------------------

def convolution(x, weight, bias=None, base_axis=1, pad=None, stride=None, dilation=None, group=1,
                channel_last=False, n_outputs=-1, outputs=None, fixed_point=None):
    """Convolution (function_bases.convolution; src/nbla/function/generic/convolution.cpp:160-197).

    fixed_point=(delta_x, delta_w): x and weight are outputs of
    fixed_point_quantize with n <= 8 and those step sizes; the convolution then
    runs on the int8 tensor-core path (exact). Otherwise full precision, for
    layers with few input channels (the network stem)."""
    if channel_last:
        raise C.NB200Error(4, "channel_last=True is not supported (nor by the reference's CPU Convolution)")
    x, weight = _check_input(x), _check_input(weight, "weight")
    bias = _check_input(bias, "bias") if bias is not None else None
    batch, Cin, H, W, Ko, kh, kw, pad, stride, dilation, out_shape = _conv_geometry(
        x, weight, bias, base_axis, pad, stride, dilation, group)
    y = torch.empty(out_shape, dtype=torch.float32, device=x.device) if outputs is None else outputs[0]
    if fixed_point is not None:
        with C.on_device(x.device):
            C.call("nb200_convolution_fxp8_f32", C.ptr(x), C.ptr(weight), C.c_float(fixed_point[0]),
                   C.c_float(fixed_point[1]), C.ptr(bias), C.ptr(y), batch, Cin, H, W, Ko, kh, kw, pad[0], pad[1],
                   stride[0], stride[1], dilation[0], dilation[1], int(group), C.stream_ptr(x.device))
        return y
    with C.on_device(x.device):
        C.call("nb200_convolution_f32", C.ptr(x), C.ptr(weight), C.ptr(bias), C.ptr(y), batch, Cin, H, W, Ko, kh, kw,
               pad[0], pad[1], stride[0], stride[1], dilation[0], dilation[1], int(group), C.stream_ptr(x.device))
    return y


def batch_normalization(x, beta, gamma, mean, variance, axes=[1], decay_rate=0.9, eps=1e-05, batch_stat=True,
                        output_stat=False, n_outputs=None):
    """Batch normalization (python/src/nnabla/functions.py batch_normalization).
    batch_stat=False: BatchNormalization::forward_impl_global
    (src/nbla/function/generic/batch_normalization.cpp:228-260). batch_stat=True: forward_impl_batch
    (:157-226): normalises with the statistics of x and updates `mean` / `variance` (the running
    statistics) in place; output_stat=True also returns the batch mean and variance."""
    x = _check_input(x)
    axes = list(axes)
    if len(axes) != 1:
        raise C.NB200Error(4, "one normalised axis is supported (got axes=%s)" % (axes,))
    ax = axes[0] + x.dim() if axes[0] < 0 else axes[0]
    Cn = int(x.shape[ax])
    outer = 1
    for s in x.shape[:ax]:
        outer *= int(s)
    inner = x.numel() // max(outer * Cn, 1)
    params = []
    for t, nm in ((beta, "beta"), (gamma, "gamma"), (mean, "mean"), (variance, "variance")):
        if t is None:
            params.append(None)
            continue
        t = _check_input(t, nm)
        if t.numel() != Cn:
            raise RuntimeError("%s must have %d elements (shape of the normalised axis)" % (nm, Cn))
        params.append(t)
    if params[2] is None or params[3] is None:
        raise RuntimeError("mean and variance are required")
    y = torch.empty_like(x)
    if batch_stat:
        bm = torch.empty(Cn, dtype=torch.float32, device=x.device)
        bv = torch.empty(Cn, dtype=torch.float32, device=x.device)
        with C.on_device(x.device):
            C.call("nb200_batch_normalization_batch_f32", C.ptr(x), C.ptr(params[0]), C.ptr(params[1]),
                   C.ptr(params[2]), C.ptr(params[3]), C.ptr(y), C.ptr(bm), C.ptr(bv), ctypes.c_int64(outer),
                   ctypes.c_int64(Cn), ctypes.c_int64(inner), C.c_float(eps), C.c_float(decay_rate), 1,
                   C.stream_ptr(x.device))
        if output_stat:
            return y, bm.reshape(params[2].shape), bv.reshape(params[3].shape)
        return y
    with C.on_device(x.device):
        C.call("nb200_batch_normalization_inference_f32", C.ptr(x), C.ptr(params[0]), C.ptr(params[1]),
               C.ptr(params[2]), C.ptr(params[3]), C.ptr(y), ctypes.c_int64(outer), ctypes.c_int64(Cn),
               ctypes.c_int64(inner), C.c_float(eps), C.stream_ptr(x.device))
    return y


def relu(x, inplace=False, n_outputs=-1, outputs=None):
    """ReLU (function_bases.relu; src/nbla/function/generic/relu.cpp)."""
    x = _check_input(x)
    y = x if inplace else _output_like(x, outputs)
    with C.on_device(x.device):
        C.call("nb200_relu_f32", C.ptr(x), C.ptr(y), C.size_t(x.numel()), C.stream_ptr(x.device))
    return y


def add2(x0, x1, inplace=False, n_outputs=-1, outputs=None):
    """Add2 (function_bases.add2; src/nbla/function/generic/add2.cpp), equal shapes."""
    x0, x1 = _check_input(x0, "x0"), _check_input(x1, "x1")
    if tuple(x0.shape) != tuple(x1.shape):
        raise C.NB200Error(4, "broadcasting add2 is not implemented: shapes %s and %s" % (tuple(x0.shape),
                                                                                         tuple(x1.shape)))
    y = x0 if inplace else _output_like(x0, outputs)
    with C.on_device(x0.device):
        C.call("nb200_add2_f32", C.ptr(x0), C.ptr(x1), C.ptr(y), C.size_t(x0.numel()), C.stream_ptr(x0.device))
    return y


def max_pooling(x, kernel, stride=None, ignore_border=True, pad=None, channel_last=False, n_outputs=-1,
                outputs=None):
    """Max pooling (function_bases.max_pooling; src/nbla/function/generic/max_pooling.cpp:140-191), 2-D."""
    if channel_last:
        raise C.NB200Error(4, "channel_last=True is not supported (nor by the reference's CPU pooling)")
    x = _check_input(x)
    kernel = tuple(kernel)
    if len(kernel) != 2:
        raise C.NB200Error(4, "2D Pooling only")
    stride = kernel if stride is None else tuple(stride)
    pad = (0, 0) if pad is None else tuple(pad)
    if len(stride) != 2 or len(pad) != 2:
        raise RuntimeError("Size of kernel and pad/stride must be same.")
    H, W = int(x.shape[-2]), int(x.shape[-1])
    maps = x.numel() // max(H * W, 1)
    Ho = (H + pad[0] - (kernel[0] - pad[0] if ignore_border else 1)) // stride[0] + 1
    Wo = (W + pad[1] - (kernel[1] - pad[1] if ignore_border else 1)) // stride[1] + 1
    y = torch.empty(tuple(x.shape[:-2]) + (Ho, Wo), dtype=torch.float32, device=x.device)
    with C.on_device(x.device):
        C.call("nb200_max_pooling_f32", C.ptr(x), C.ptr(y), ctypes.c_int64(maps), H, W, kernel[0], kernel[1],
               stride[0], stride[1], pad[0], pad[1], int(bool(ignore_border)), C.stream_ptr(x.device))
    return y


def global_average_pooling(x, n_outputs=-1, outputs=None):
    """Global average pooling (function_bases.global_average_pooling;
    src/nbla/function/generic/global_average_pooling.cpp): [N, C, ...] -> [N, C, 1, 1]."""
    x = _check_input(x)
    if x.dim() < 2:
        raise RuntimeError("GlobalAveragePooling averages across the channel, so the input's shape must have a "
                           "dimension equal to or larger than 2. actual: %d" % x.dim())
    N, Cn = int(x.shape[0]), int(x.shape[1])
    S = x.numel() // max(N * Cn, 1)
    y = torch.empty((N, Cn, 1, 1), dtype=torch.float32, device=x.device)
    with C.on_device(x.device):
        C.call("nb200_global_average_pooling_f32", C.ptr(x), C.ptr(y), ctypes.c_int64(N * Cn), ctypes.c_int64(S),
               C.stream_ptr(x.device))
    return y


class INQState:
    """What one INQAffine function instance keeps across forward passes (inq_affine.cpp:74-80): the
    weights and indicators of the previous pass, the pass counter, the random stream."""

    def __init__(self, weight, seed=-1):
        self.old_weights = torch.zeros_like(weight)
        self.old_indicators = torch.zeros(weight.shape, dtype=torch.int32, device=weight.device)
        self.counter = 0
        self.generator = None
        if seed != -1:
            self.generator = torch.Generator(device=weight.device)
            self.generator.manual_seed(int(seed))


def inq_update_weights(weight, indicators, state, num_bits=4, inq_iterations=(), selection_algorithm="largest_abs"):
    """The weight update of INQAffine / INQConvolution (inq_affine.cpp:82-203), in place on `weight` (fp32)
    and `indicators` (int32). The selection step runs on the device through torch's sort / Bernoulli
    sampler; the random stream is torch's, not the reference's mt19937."""
    if selection_algorithm not in ("largest_abs", "random"):
        raise ValueError('Provided value for selection algorithm not valid: %s. Valid values are "largest_abs" '
                         'and "random".' % selection_algorithm)
    weight = _check_input(weight, "weight")
    if indicators.dtype != torch.int32 or indicators.shape != weight.shape or not indicators.is_contiguous():
        raise RuntimeError("Indicators and weights must have same size (indicators as contiguous int32).")
    n = weight.numel()
    its = [int(v) for v in inq_iterations]
    with C.on_device(weight.device):
        C.call("nb200_inq_restore_f32", C.ptr(weight), C.ptr(state.old_weights), C.ptr(state.old_indicators),
               C.size_t(n), C.stream_ptr(weight.device))
    fix_all = 0
    if state.counter in its:
        if its[-1] == state.counter:
            fix_all = 1
        elif selection_algorithm == "largest_abs":
            flat = indicators.view(-1)
            order = torch.argsort(weight.abs().view(-1), descending=True, stable=True)
            learnable = flat[order] == 0
            k = int(learnable.sum().item()) // 2
            if k == 0:  # the reference's loop looks at the largest weight once before it stops (:131-139)
                chosen = order[:1][learnable[:1]]
            else:
                chosen = order[learnable & (torch.cumsum(learnable, 0) <= k)]
            flat[chosen] = 1
        else:
            flat = indicators.view(-1)
            draws = torch.bernoulli(torch.full((n,), 0.5, device=weight.device), generator=state.generator).to(torch.int32)
            flat.copy_(torch.where(flat == 0, draws, flat))
    with C.on_device(weight.device):
        C.call("nb200_inq_quantize_f32", C.ptr(weight), C.ptr(indicators), C.ptr(state.old_weights),
               C.ptr(state.old_indicators), C.size_t(n), int(num_bits), fix_all, C.stream_ptr(weight.device))
    state.counter += 1


def inq_affine(x, weight, indicator_fixedweights, bias=None, base_axis=1, num_bits=4, inq_iterations=(),
               selection_algorithm="largest_abs", seed=-1, state=None):
    """INQ Affine (python/src/nnabla/functions.py inq_affine; src/nbla/function/generic/inq_affine.cpp:82-203):
    updates `weight` and `indicator_fixedweights` in place, then the affine. `state` (INQState) stands for the
    function instance, which in nnabla carries the previous weights, indicators and the pass counter."""
    if state is None:
        raise RuntimeError("inq_affine needs the INQState of its layer (the reference keeps it in the function)")
    inq_update_weights(weight, indicator_fixedweights, state, num_bits, inq_iterations, selection_algorithm)
    return affine(x, weight, bias, base_axis)


def inq_convolution(x, weight, indicator_fixedweights, bias=None, base_axis=1, pad=None, stride=None, dilation=None,
                    group=1, num_bits=4, inq_iterations=(), selection_algorithm="largest_abs", seed=-1, state=None):
    """INQ Convolution (src/nbla/function/generic/inq_convolution.cpp:86-204): INQAffine's weight update, in
    place, then the convolution."""
    if state is None:
        raise RuntimeError("inq_convolution needs the INQState of its layer (the reference keeps it in the function)")
    inq_update_weights(weight, indicator_fixedweights, state, num_bits, inq_iterations, selection_algorithm)
    return convolution(x, weight, bias, base_axis, pad, stride, dilation, group)


def _grad_out(like, accum, dx):
    if dx is None:
        if accum:
            raise RuntimeError("accum needs the gradient buffer to add to")
        return torch.empty_like(like)
    return _check_input(dx, "dx")


def batch_normalization_backward(x, dy, gamma, mean, variance, axes=[1], eps=1e-05, batch_stat=True, dmean=None,
                                 dvar=None, propagate_down=(True, True, True), accum=(False, False, False),
                                 grads=(None, None, None)):
    """BatchNormalization::backward_impl (batch_normalization.cpp:262-486). mean / variance: the batch
    statistics the forward pass returned (batch_stat) or the running ones. Returns (dx, dbeta, dgamma),
    None where propagate_down is False."""
    x, dy = _check_input(x), _check_input(dy, "dy")
    axes = list(axes)
    if len(axes) != 1:
        raise C.NB200Error(4, "one normalised axis is supported (got axes=%s)" % (axes,))
    ax = axes[0] + x.dim() if axes[0] < 0 else axes[0]
    Cn = int(x.shape[ax])
    outer = 1
    for s_ in x.shape[:ax]:
        outer *= int(s_)
    inner = x.numel() // max(outer * Cn, 1)
    dx = _grad_out(x, accum[0], grads[0]) if propagate_down[0] else None
    like = torch.empty(Cn, dtype=torch.float32, device=x.device)
    db = _grad_out(like, accum[1], grads[1]) if propagate_down[1] else None
    dg = _grad_out(like, accum[2], grads[2]) if propagate_down[2] else None
    with C.on_device(x.device):
        C.call("nb200_batch_normalization_backward_f32", C.ptr(x), C.ptr(dy), C.ptr(gamma), C.ptr(mean),
               C.ptr(variance), C.ptr(dmean), C.ptr(dvar), C.ptr(dx), C.ptr(db), C.ptr(dg), ctypes.c_int64(outer),
               ctypes.c_int64(Cn), ctypes.c_int64(inner), C.c_float(eps), int(bool(batch_stat)), int(bool(accum[0])),
               int(bool(accum[1])), int(bool(accum[2])), C.stream_ptr(x.device))
    return dx, db, dg


def relu_backward(y, dy, accum=False, dx=None):
    """ReLU::backward_impl (relu.cpp:41-66); y is the forward output."""
    y, dy = _check_input(y), _check_input(dy, "dy")
    dx = _grad_out(y, accum, dx)
    with C.on_device(y.device):
        C.call("nb200_relu_backward_f32", C.ptr(y), C.ptr(dy), C.ptr(dx), C.size_t(y.numel()), int(bool(accum)),
               C.stream_ptr(y.device))
    return dx


def add2_backward(dy, accum=False, dx=None):
    """Add2::backward_impl for one input of equal shape: dx (+)= dy."""
    dy = _check_input(dy, "dy")
    dx = _grad_out(dy, accum, dx)
    with C.on_device(dy.device):
        C.call("nb200_add2_backward_f32", C.ptr(dy), C.ptr(dx), C.size_t(dy.numel()), int(bool(accum)),
               C.stream_ptr(dy.device))
    return dx


def global_average_pooling_backward(x_shape, dy, accum=False, dx=None):
    """GlobalAveragePooling::backward_impl (global_average_pooling.cpp:75-117)."""
    dy = _check_input(dy, "dy")
    N, Cn = int(x_shape[0]), int(x_shape[1])
    S = 1
    for s_ in x_shape[2:]:
        S *= int(s_)
    dx = _grad_out(torch.empty(tuple(x_shape), dtype=torch.float32, device=dy.device), accum, dx)
    with C.on_device(dy.device):
        C.call("nb200_global_average_pooling_backward_f32", C.ptr(dy), C.ptr(dx), ctypes.c_int64(N * Cn),
               ctypes.c_int64(S), int(bool(accum)), C.stream_ptr(dy.device))
    return dx


def max_pooling_backward(x, dy, kernel, stride=None, ignore_border=True, pad=None, accum=False, dx=None):
    """MaxPooling::backward_impl (max_pooling.cpp:194-228); x is the forward input."""
    x, dy = _check_input(x), _check_input(dy, "dy")
    stride = tuple(kernel) if stride is None else tuple(stride)
    pad = (0, 0) if pad is None else tuple(pad)
    H, W = int(x.shape[-2]), int(x.shape[-1])
    maps = x.numel() // max(H * W, 1)
    dx = _grad_out(x, accum, dx)
    with C.on_device(x.device):
        C.call("nb200_max_pooling_backward_f32", C.ptr(x), C.ptr(dy), C.ptr(dx), ctypes.c_int64(maps), H, W,
               int(kernel[0]), int(kernel[1]), int(stride[0]), int(stride[1]), int(pad[0]), int(pad[1]),
               int(bool(ignore_border)), int(bool(accum)), C.stream_ptr(x.device))
    return dx


def bn_add_relu_fixed_point(a, bn_a, b=None, bn_b=None, eps=1e-05, relu=True, quantize=True, sign=True, n=8,
                            delta=2 ** -4, outputs=None):
    """Inference-time fusion: fixed_point_quantize(relu(batch_normalization(a) [+ batch_normalization(b) | + b]))
    in one pass, bit-identical to the separate functions.

    bn_a / bn_b are (beta, gamma, mean, variance) tuples over axis 1 (bn_b=None
    adds b as it is, b=None leaves the second term out). The reference's fused
    form of the first three stages is FusedBatchNormalization
    (src/nbla/function/generic/fused_batch_normalization.cpp)."""
    a = _check_input(a, "a")
    if a.dim() < 2:
        raise RuntimeError("the normalised axis is axis 1")
    Cn = int(a.shape[1])
    outer, inner = int(a.shape[0]), a.numel() // max(int(a.shape[0]) * Cn, 1)

    def params(t4, what):
        out = []
        for t, nm in zip(t4, ("beta", "gamma", "mean", "variance")):
            if t is None:
                if nm in ("mean", "variance"):
                    raise RuntimeError("mean and variance are required (%s)" % what)
                out.append(None)
                continue
            t = _check_input(t, nm)
            if t.numel() != Cn:
                raise RuntimeError("%s must have %d elements (shape of the normalised axis)" % (nm, Cn))
            out.append(t)
        return out
    pa = params(bn_a, "a")
    pb = [None] * 4
    if b is not None:
        b = _check_input(b, "b")
        _same_shape(a, b, "a vs b")
        if bn_b is not None:
            pb = params(bn_b, "b")
    elif bn_b is not None:
        raise RuntimeError("bn_b without b")
    y = _output_like(a, outputs)
    with C.on_device(a.device):
        C.call("nb200_bn_add_relu_fxp_f32", C.ptr(a), C.ptr(pa[0]), C.ptr(pa[1]), C.ptr(pa[2]), C.ptr(pa[3]),
               C.ptr(b), C.ptr(pb[0]), C.ptr(pb[1]), C.ptr(pb[2]), C.ptr(pb[3]), C.ptr(y), ctypes.c_int64(outer),
               ctypes.c_int64(Cn), ctypes.c_int64(inner), C.c_float(eps), int(bool(relu)), int(bool(quantize)),
               int(bool(sign)), int(n), C.c_float(delta), C.stream_ptr(a.device))
    return y


# ---------------------------------------------------------------------------
# Activations kept as int8 channel-last codes between layers
# ---------------------------------------------------------------------------

def codes_nhwc_slots(channels, group=1):
    """Slots per pixel of a codes tensor for `channels` channels in `group` groups."""
    fn = C.lib().nb200_codes_nhwc_slots
    fn.restype = ctypes.c_int64
    n = int(fn(ctypes.c_int64(int(channels)), int(group)))
    if n <= 0:
        raise RuntimeError("Number of input channel needs to be divisible by group. Input channel: %d, group: %d."
                           % (channels, group))
    return n


def _nchw_extents(x):
    if x.dim() < 2:
        raise RuntimeError("the channel axis is axis 1")
    batch, ch = int(x.shape[0]), int(x.shape[1])
    return batch, ch, x.numel() // max(batch * ch, 1)


def fixed_point_codes_nhwc(xq, delta=2 ** -4, group=1):
    """xq [batch, channels, ...] (an output of fixed_point_quantize with step
    `delta` and n <= 8) -> int8 codes [batch, inner, slots], channel-last."""
    xq = _check_input(xq, "xq")
    batch, ch, inner = _nchw_extents(xq)
    codes = torch.empty((batch, inner, codes_nhwc_slots(ch, group)), dtype=torch.int8, device=xq.device)
    with C.on_device(xq.device):
        C.call("nb200_fixed_point_codes_nhwc", C.ptr(xq), C.ptr(codes), ctypes.c_int64(batch), ctypes.c_int64(ch),
               ctypes.c_int64(inner), int(group), C.c_float(delta), C.stream_ptr(xq.device))
    return codes


def _check_codes(codes, batch, inner, channels, group, name="codes"):
    if not isinstance(codes, torch.Tensor) or not codes.is_cuda or codes.dtype != torch.int8:
        raise TypeError("%s must be an int8 torch.Tensor on a CUDA device" % name)
    want = (batch, inner, codes_nhwc_slots(channels, group))
    if tuple(codes.shape) != want or not codes.is_contiguous():
        raise RuntimeError("%s must be a contiguous [batch, inner, slots] = %s tensor, got %s"
                           % (name, want, tuple(codes.shape)))
    return codes


def codes_nhwc_to_float(codes, shape, delta=2 ** -4, group=1):
    """codes [batch, inner, slots] -> fp32 tensor of `shape` = [batch, channels, ...] holding code * delta."""
    shape = tuple(int(v) for v in shape)
    batch, ch = shape[0], shape[1]
    inner = 1
    for v in shape[2:]:
        inner *= v
    codes = _check_codes(codes, batch, inner, ch, group)
    y = torch.empty(shape, dtype=torch.float32, device=codes.device)
    with C.on_device(codes.device):
        C.call("nb200_codes_nhwc_to_f32", C.ptr(codes), C.ptr(y), ctypes.c_int64(batch), ctypes.c_int64(ch),
               ctypes.c_int64(inner), int(group), C.c_float(delta), C.stream_ptr(codes.device))
    return y


def bn_add_relu_fixed_point_codes(a, bn_a, b=None, bn_b=None, b_codes=None, b_delta=None, eps=1e-05, relu=True,
                                  sign=True, n=8, delta=2 ** -4, group=1):
    """bn_add_relu_fixed_point whose result is returned as int8 channel-last
    codes (value = code * delta). The second operand is b (fp32, shaped like
    a, normalised with bn_b when given) or b_codes (codes of a tensor shaped
    like a, step b_delta, default delta)."""
    a = _check_input(a, "a")
    batch, Cn, inner = _nchw_extents(a)

    def params(t4, what):
        out = []
        for t, nm in zip(t4, ("beta", "gamma", "mean", "variance")):
            if t is None:
                if nm in ("mean", "variance"):
                    raise RuntimeError("mean and variance are required (%s)" % what)
                out.append(None)
                continue
            t = _check_input(t, nm)
            if t.numel() != Cn:
                raise RuntimeError("%s must have %d elements (shape of the normalised axis)" % (nm, Cn))
            out.append(t)
        return out
    pa = params(bn_a, "a")
    pb = [None] * 4
    if b is not None and b_codes is not None:
        raise RuntimeError("the second operand is either b or b_codes")
    if b is not None:
        b = _check_input(b, "b")
        _same_shape(a, b, "a vs b")
        if bn_b is not None:
            pb = params(bn_b, "b")
    elif bn_b is not None:
        raise RuntimeError("bn_b without b")
    if b_codes is not None:
        b_codes = _check_codes(b_codes, batch, inner, Cn, group, "b_codes")
    y = torch.empty((batch, inner, codes_nhwc_slots(Cn, group)), dtype=torch.int8, device=a.device)
    with C.on_device(a.device):
        C.call("nb200_bn_add_relu_fxp_codes_nhwc", C.ptr(a), C.ptr(pa[0]), C.ptr(pa[1]), C.ptr(pa[2]), C.ptr(pa[3]),
               C.ptr(b), C.ptr(pb[0]), C.ptr(pb[1]), C.ptr(pb[2]), C.ptr(pb[3]), C.ptr(b_codes),
               C.c_float(delta if b_delta is None else b_delta), C.ptr(y), ctypes.c_int64(batch), ctypes.c_int64(Cn),
               ctypes.c_int64(inner), int(group), C.c_float(eps), int(bool(relu)), int(bool(sign)), int(n),
               C.c_float(delta), C.stream_ptr(a.device))
    return y


def max_pooling_codes(codes, shape, kernel, stride=None, ignore_border=True, pad=None, group=1):
    """max_pooling on int8 channel-last codes of a tensor of `shape` = (batch,
    channels, height, width); returns (codes [batch, Ho * Wo, slots], pooled shape).
    The maximum of the codes is the code of the maximum (python/src/nnabla/functions.py max_pooling;
    src/nbla/function/generic/max_pooling.cpp:140-191)."""
    shape = tuple(int(v) for v in shape)
    if len(shape) != 4:
        raise C.NB200Error(4, "only [batch, channels, height, width] tensors are implemented")
    batch, Cn, H, W = shape
    codes = _check_codes(codes, batch, H * W, Cn, group)
    kernel = tuple(kernel)
    stride = kernel if stride is None else tuple(stride)
    pad = (0, 0) if pad is None else tuple(pad)
    Ho = (H + pad[0] - (kernel[0] - pad[0] if ignore_border else 1)) // stride[0] + 1
    Wo = (W + pad[1] - (kernel[1] - pad[1] if ignore_border else 1)) // stride[1] + 1
    if Ho <= 0 or Wo <= 0:
        raise RuntimeError("pooling output would be empty")
    y = torch.empty((batch, Ho * Wo, codes.shape[2]), dtype=torch.int8, device=codes.device)
    with C.on_device(codes.device):
        C.call("nb200_max_pooling_codes_nhwc", C.ptr(codes), C.ptr(y), ctypes.c_int64(batch), ctypes.c_int64(Cn), H, W,
               int(group), int(kernel[0]), int(kernel[1]), int(stride[0]), int(stride[1]), int(pad[0]), int(pad[1]),
               int(bool(ignore_border)), C.stream_ptr(codes.device))
    return y, (batch, Cn, Ho, Wo)


def binary_weight_convolution_from_codes(x_codes, x_shape, weight, binary_weight, alpha, bias=None, pad=None,
                                         stride=None, dilation=None, group=1, quantize_zero_to=1.0,
                                         activation_delta=2 ** -4, outputs=None):
    """binary_weight_convolution (binary_connect_convolution when alpha is
    None) on activations given as int8 channel-last codes of a tensor of shape
    x_shape = (batch, channels, height, width) with step activation_delta."""
    weight = _check_input(weight, "weight")
    binary_weight = _check_input(binary_weight, "binary_weight")
    bias = _check_input(bias, "bias") if bias is not None else None
    x_shape = tuple(int(v) for v in x_shape)
    if len(x_shape) != 4:
        raise C.NB200Error(4, "only 2-D convolution with one batch axis is implemented for code tensors")
    like = torch.empty(x_shape, dtype=torch.float32, device="meta")
    batch, Cin, H, W, Ko, kh, kw, pad, stride, dilation, out_shape = _conv_geometry(
        like, weight, bias, 1, pad, stride, dilation, group)
    x_codes = _check_codes(x_codes, batch, H * W, Cin, group, "x_codes")
    _same_shape(weight, binary_weight, "float vs binary")
    if alpha is not None:
        alpha = _check_input(alpha, "alpha")
        if alpha.numel() != Ko:
            raise RuntimeError("Size of alpha must be equal to the number of output maps.")
    y = torch.empty(out_shape, dtype=torch.float32, device=weight.device) if outputs is None else outputs[0]
    with C.on_device(weight.device):
        C.call("nb200_binary_convolution_codes_f32", C.ptr(x_codes), C.ptr(weight), C.ptr(binary_weight),
               C.ptr(alpha), C.ptr(bias), C.ptr(y), batch, Cin, H, W, Ko, kh, kw, pad[0], pad[1], stride[0],
               stride[1], dilation[0], dilation[1], int(group), C.c_float(quantize_zero_to),
               C.c_float(activation_delta), C.stream_ptr(weight.device))
    return y


class PreparedBinaryWeights:
    """sign(w), alpha and the int8 side-band of a binary convolution, made once
    per weight update (prepare_binary_weights)."""

    def __init__(self, shape, group, binary_weight, alpha, side):
        self.shape, self.group = tuple(shape), int(group)
        self.binary_weight, self.alpha, self.side = binary_weight, alpha, side


def prepare_binary_weights(weight, group=1, quantize_zero_to=1.0, with_alpha=True):
    """Binarises `weight` [outmaps, channels / group, kh, kw] once: what the binary
    convolutions otherwise redo on every call (binary_weight_convolution.cpp:72-117).
    with_alpha=False gives BinaryConnect weights (no scaling)."""
    weight = _check_input(weight, "weight")
    if weight.dim() != 4:
        raise C.NB200Error(4, "only 2-D convolution weights are implemented")
    Ko, Cg, kh, kw = (int(v) for v in weight.shape)
    fn = C.lib().nb200_binary_weights_side_bytes
    fn.restype = ctypes.c_int64
    nbytes = int(fn(Ko, Cg * int(group), kh, kw, int(group)))
    if nbytes <= 0 or Ko % group != 0:
        raise RuntimeError("Number of output channel needs to be divisible by group. Output channel: %d, group: %d."
                           % (Ko, group))
    wb = torch.empty_like(weight)
    alpha = torch.empty((Ko,), dtype=torch.float32, device=weight.device) if with_alpha else None
    side = torch.empty((nbytes,), dtype=torch.int8, device=weight.device)
    with C.on_device(weight.device):
        C.call("nb200_binary_weights_prepare_i8", C.ptr(weight), C.ptr(wb), C.ptr(alpha), C.ptr(side), Ko,
               Cg * int(group), kh, kw, int(group), C.c_float(quantize_zero_to), C.stream_ptr(weight.device))
    return PreparedBinaryWeights(weight.shape, group, wb, alpha, side)


def binary_convolution_from_codes_prepared(x_codes, x_shape, prepared, bias=None, pad=None, stride=None,
                                           dilation=None, activation_delta=2 ** -4, outputs=None):
    """binary_weight_convolution_from_codes with weights from prepare_binary_weights."""
    bias = _check_input(bias, "bias") if bias is not None else None
    x_shape = tuple(int(v) for v in x_shape)
    if len(x_shape) != 4:
        raise C.NB200Error(4, "only 2-D convolution with one batch axis is implemented for code tensors")
    like_x = torch.empty(x_shape, dtype=torch.float32, device="meta")
    like_w = torch.empty(prepared.shape, dtype=torch.float32, device="meta")
    batch, Cin, H, W, Ko, kh, kw, pad, stride, dilation, out_shape = _conv_geometry(
        like_x, like_w, bias, 1, pad, stride, dilation, prepared.group)
    x_codes = _check_codes(x_codes, batch, H * W, Cin, prepared.group, "x_codes")
    dev = x_codes.device
    y = torch.empty(out_shape, dtype=torch.float32, device=dev) if outputs is None else outputs[0]
    with C.on_device(dev):
        C.call("nb200_binary_convolution_codes_prepared_f32", C.ptr(x_codes), C.ptr(prepared.side),
               C.ptr(prepared.alpha), C.ptr(bias), C.ptr(y), batch, Cin, H, W, Ko, kh, kw, pad[0], pad[1], stride[0],
               stride[1], dilation[0], dilation[1], int(prepared.group), C.c_float(activation_delta),
               C.stream_ptr(dev))
    return y


# ---------------------------------------------------------------------------
# Layers with batch normalization folded in (inference)
# ---------------------------------------------------------------------------

def convolution_codes_folded(x_codes, x_shape, prepared, scale, bias=None, pad=None, stride=None, dilation=None,
                             residual_codes=None, residual_delta=None, residual=None, relu=True, sign=True, n=8,
                             delta=2 ** -4, output="codes"):
    """A binary-weight convolution whose BatchNormalization was folded into a per-map factor and
    bias (batch_normalization_folding.py:92-200), with Add2 of the residual, ReLU and
    FixedPointQuantize in the convolution's epilogue.

    x_codes: int8 channel-last codes of a tensor of shape x_shape; prepared: prepare_binary_weights;
    scale [outmaps] = alpha * c0 * (step of x_codes), bias [outmaps] = c1; residual_codes (with
    residual_delta) or residual (fp32 channel-last [batch, Ho * Wo, slots]) is added before the ReLU.
    output="codes": int8 codes [batch, Ho * Wo, slots]; output="float": the fp32 value before ReLU
    and quantizer, channel-last (what a shortcut branch hands to the main branch's epilogue).
    Returns (result, (batch, outmaps, Ho, Wo))."""
    if prepared.group != 1:
        raise C.NB200Error(4, "grouped convolutions are not supported by the folded code path")
    scale = _check_input(scale, "scale")
    bias = _check_input(bias, "bias") if bias is not None else None
    x_shape = tuple(int(v) for v in x_shape)
    if len(x_shape) != 4:
        raise C.NB200Error(4, "only 2-D convolution with one batch axis is implemented for code tensors")
    like_x = torch.empty(x_shape, dtype=torch.float32, device="meta")
    like_w = torch.empty(prepared.shape, dtype=torch.float32, device="meta")
    batch, Cin, H, W, Ko, kh, kw, pad, stride, dilation, out_shape = _conv_geometry(
        like_x, like_w, bias, 1, pad, stride, dilation, 1)
    x_codes = _check_codes(x_codes, batch, H * W, Cin, 1, "x_codes")
    if scale.numel() != Ko:
        raise RuntimeError("Size of scale must be equal to the number of output maps.")
    dev = x_codes.device
    Ho, Wo = out_shape[2], out_shape[3]
    slots = codes_nhwc_slots(Ko, 1)
    if residual_codes is not None:
        residual_codes = _check_codes(residual_codes, batch, Ho * Wo, Ko, 1, "residual_codes")
    if residual is not None and tuple(residual.shape) != (batch, Ho * Wo, slots):
        raise RuntimeError("residual must be channel-last fp32 of shape %s" % ((batch, Ho * Wo, slots),))
    y_codes = y_f32 = None
    if output == "codes":
        y_codes = torch.empty((batch, Ho * Wo, slots), dtype=torch.int8, device=dev)
    elif output == "float":
        y_f32 = torch.empty((batch, Ho * Wo, slots), dtype=torch.float32, device=dev)
    else:
        raise ValueError("output must be 'codes' or 'float'")
    with C.on_device(dev):
        C.call("nb200_convolution_codes_folded_nhwc", C.ptr(x_codes), C.ptr(prepared.side), C.ptr(scale), C.ptr(bias),
               C.ptr(residual_codes), C.c_float(residual_delta or 0.0), C.ptr(residual), C.ptr(y_codes), C.ptr(y_f32),
               batch, Cin, H, W, Ko, kh, kw, pad[0], pad[1], stride[0], stride[1], dilation[0], dilation[1],
               int(bool(relu)), int(bool(sign)), int(n), C.c_float(delta), C.stream_ptr(dev))
    return (y_codes if y_codes is not None else y_f32), tuple(out_shape)


def convolution_relu_fixed_point_codes(x, weight, bias=None, pad=None, stride=None, relu=True, sign=True, n=8,
                                       delta=2 ** -4):
    """Full-precision convolution of an input with few channels (a network stem, weights and bias
    with BatchNormalization folded in), ReLU and FixedPointQuantize in one kernel; the result is
    int8 channel-last codes. Returns (codes [batch, Ho * Wo, slots], (batch, outmaps, Ho, Wo))."""
    x, weight = _check_input(x), _check_input(weight, "weight")
    bias = _check_input(bias, "bias") if bias is not None else None
    batch, Cin, H, W, Ko, kh, kw, pad, stride, dilation, out_shape = _conv_geometry(
        x, weight, bias, 1, pad, stride, None, 1)
    slots = codes_nhwc_slots(Ko, 1)
    y = torch.empty((batch, out_shape[2] * out_shape[3], slots), dtype=torch.int8, device=x.device)
    with C.on_device(x.device):
        C.call("nb200_convolution_relu_fxp_codes_nhwc", C.ptr(x), C.ptr(weight), C.ptr(bias), C.ptr(y), batch, Cin, H,
               W, Ko, kh, kw, pad[0], pad[1], stride[0], stride[1], int(bool(relu)), int(bool(sign)), int(n),
               C.c_float(delta), C.stream_ptr(x.device))
    return y, tuple(out_shape)


def global_average_pooling_codes(codes, shape, delta=2 ** -4):
    """GlobalAveragePooling of a tensor held as channel-last codes: [batch, channels, 1, 1] fp32."""
    return global_average_pooling(codes_nhwc_to_float(codes, shape, delta))


# ---------------------------------------------------------------------------
# Sibling quantization functions
# ---------------------------------------------------------------------------

def _unary(entry, x, outputs):
    x = _check_input(x)
    y = _output_like(x, outputs)
    with C.on_device(x.device):
        C.call(entry, C.ptr(x), C.ptr(y), C.size_t(x.numel()), C.stream_ptr(x.device))
    return y


def binary_sigmoid(x, n_outputs=-1, outputs=None):
    """Element-wise binary sigmoid, 1 where x > 0 and 0 elsewhere
    (python/src/nnabla/functions.py binary_sigmoid; include/nbla/function/binary_sigmoid.hpp:50-52)."""
    return _unary("nb200_binary_sigmoid_f32", x, outputs)


def binary_tanh(x, n_outputs=-1, outputs=None):
    """Element-wise binary tanh, 1 where x > 0 and -1 elsewhere (include/nbla/function/binary_tanh.hpp:51-52)."""
    return _unary("nb200_binary_tanh_f32", x, outputs)


def _unary_backward(entry, x, dy, accum, dx):
    x, dy, dx = _grad_buffers(x, dy, dx, accum)
    with C.on_device(x.device):
        C.call(entry, C.ptr(x), C.ptr(dy), C.ptr(dx), C.size_t(x.numel()), int(bool(accum)), C.stream_ptr(x.device))
    return dx


def binary_sigmoid_backward(x, dy, accum=False, dx=None):
    return _unary_backward("nb200_binary_sigmoid_backward_f32", x, dy, accum, dx)


def binary_tanh_backward(x, dy, accum=False, dx=None):
    return _unary_backward("nb200_binary_tanh_backward_f32", x, dy, accum, dx)


_ROUND_MODES = {"HALF_AWAY_FROM_ZERO": 0, "HALF_TO_EVEN": 1}
_QL_DTYPES = {1: 1, 2: 2, "int8": 1, "uint8": 2, torch.int8: 1, torch.uint8: 2}


def _linear_params(x, scale, zero_point):
    x, scale = _check_input(x), _check_input(scale, "scale")
    zero_point = _check_input(zero_point, "zero_point") if zero_point is not None else None
    for t in (scale, zero_point):
        if t is not None and t.dim() != x.dim():
            raise RuntimeError("Dimensions of inputs must be same (%d, %d)." % (x.dim(), t.dim()))
    return x, scale, zero_point


def quantize_linear(x, scale, zero_point, round_mode="HALF_AWAY_FROM_ZERO", narrow_range=False, dtype=1, n_outputs=-1,
                    outputs=None):
    """saturate(round(x / scale) + zero_point) (python/src/nnabla/functions.py quantize_linear;
    src/nbla/function/generic/quantize_linear.cpp:103-122). As in the reference
    zero_point is rounded and saturated IN PLACE. dtype: 1 / "int8" = BYTE, 2 / "uint8" = UBYTE."""
    x, scale, zero_point = _linear_params(x, scale, zero_point)
    if round_mode not in _ROUND_MODES:
        raise RuntimeError("round_mode must be HALF_AWAY_FROM_ZERO or HALF_TO_EVEN")
    if dtype not in _QL_DTYPES:
        raise C.NB200Error(4, "dtype must be int8 (BYTE) or uint8 (UBYTE)")
    y = _output_like(x, outputs)
    with C.on_device(x.device):
        C.call("nb200_quantize_linear_f32", C.ptr(x), C.i64_array(x.shape), int(x.dim()), C.ptr(scale),
               C.i64_array(scale.shape), C.ptr(zero_point), C.i64_array(zero_point.shape), C.ptr(y),
               _ROUND_MODES[round_mode], int(bool(narrow_range)), _QL_DTYPES[dtype], C.stream_ptr(x.device))
    return y


def dequantize_linear(x, scale, zero_point, n_outputs=-1, outputs=None):
    """(x - zero_point) * scale (src/nbla/function/generic/dequantize_linear.cpp:60-71)."""
    x, scale, zero_point = _linear_params(x, scale, zero_point)
    y = _output_like(x, outputs)
    with C.on_device(x.device):
        C.call("nb200_dequantize_linear_f32", C.ptr(x), C.i64_array(x.shape), int(x.dim()), C.ptr(scale),
               C.i64_array(scale.shape), C.ptr(zero_point), C.i64_array(zero_point.shape), C.ptr(y),
               C.stream_ptr(x.device))
    return y


def _linear_backward(entry, dy, scale, accum, dx):
    dy, scale, _ = _linear_params(dy, scale, None)
    _, dy, dx = _grad_buffers(dy, dy, dx, accum)
    with C.on_device(dy.device):
        C.call(entry, C.ptr(dy), C.i64_array(dy.shape), int(dy.dim()), C.ptr(scale), C.i64_array(scale.shape),
               C.ptr(dx), int(bool(accum)), C.stream_ptr(dy.device))
    return dx


def quantize_linear_backward(dy, scale, accum=False, dx=None):
    """dx (+)= dy / scale (quantize_linear.cpp:137-147); the reference has no gradient for scale or zero point."""
    return _linear_backward("nb200_quantize_linear_backward_f32", dy, scale, accum, dx)


def dequantize_linear_backward(dy, scale, accum=False, dx=None):
    """dx (+)= dy * scale (dequantize_linear.cpp:92-102)."""
    return _linear_backward("nb200_dequantize_linear_backward_f32", dy, scale, accum, dx)


def prune(x, rate=0.9, n_outputs=-1, outputs=None):
    """Prune the input: values whose magnitude is below the rate-quantile of
    |x| become zero (python/src/nnabla/functions.py prune; src/nbla/function/generic/prune.cpp:38-72)."""
    x = _check_input(x)
    y = _output_like(x, outputs)
    with C.on_device(x.device):
        C.call("nb200_prune_f32", C.ptr(x), C.ptr(y), C.size_t(x.numel()), C.c_float(rate), C.stream_ptr(x.device))
    return y


def prune_backward(dy, accum=False, dx=None):
    """Prune::backward_impl (prune.cpp:74-88): the gradient passes unchanged."""
    _, dy, dx = _grad_buffers(dy, dy, dx, accum)
    with C.on_device(dy.device):
        C.call("nb200_prune_backward_f32", C.ptr(dy), C.ptr(dx), C.size_t(dy.numel()), int(bool(accum)),
               C.stream_ptr(dy.device))
    return dx
