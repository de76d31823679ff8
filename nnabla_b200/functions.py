"""Host-side mirror of nnabla's function API for the quantized-layer forward path.

Same names, argument order, defaults and error behaviour as
python/src/nnabla/functions.py:416-692 (quantizers) and the generated
function_bases for the binary layers, so code and tests written against
`nnabla.functions` read the same here. Arrays are torch CUDA tensors (torch
only provides device memory and streams); every computation is one call into
libnnabla_b200.so. There is no CPU path.
"""
import ctypes

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
    if y.shape != x.shape or y.dtype != x.dtype or y.device != x.device or not y.is_contiguous():
        raise RuntimeError("outputs[0] must be a contiguous tensor of x's shape, dtype and device")
    return y


def fixed_point_quantize(x, sign=True, n=8, delta=2 ** -4, quantize=True, ste_fine_grained=True, outputs=None):
    """Fixed Point Quantize (python/src/nnabla/functions.py:416-482).

    Forward of FixedPointQuantize (src/nbla/function/generic/fixed_point_quantize.cpp:45-66).
    """
    if not quantize:
        return x
    x = _check_input(x)
    y = _output_like(x, outputs)
    with torch.cuda.device(x.device):
        C.call("nb200_fixed_point_quantize_f32", C.ptr(x), C.ptr(y), C.size_t(x.numel()), int(bool(sign)), int(n),
               C.c_float(delta), C.stream_ptr(x.device))
    return y


def fixed_point_quantize_with_codes(x, sign=True, n=8, delta=2 ** -4):
    """fixed_point_quantize that also returns the int8 codes k (y = k * delta)."""
    x = _check_input(x)
    y = torch.empty_like(x)
    codes = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    with torch.cuda.device(x.device):
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
    with torch.cuda.device(x.device):
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
    with torch.cuda.device(x.device):
        C.call("nb200_min_max_quantize_f32", C.ptr(x), C.i64_array(x.shape), int(x.dim()), C.ptr(qs[0]),
               C.ptr(qs[1]), C.ptr(qs[2]), C.ptr(qs[3]), C.i64_array(qs[0].shape), C.c_float(decay),
               int(bool(x_min_max)), int(bool(ema)), C.c_float(eps), C.ptr(y), ctypes.c_void_p(0),
               C.stream_ptr(x.device))
    return y
