"""Host-side mirror of `nnabla.parametric_functions` for the quantized-layer path.

Same function names, argument order, defaults and parameter names ("W", "Wb",
"alpha", "b", "beta", "gamma", "mean", "var" under the scopes "bwn_conv",
"bwn_affine", "bicon_conv", "bicon_affine", "inq_conv", "inq_affine", "conv", "affine", "bn") as
python/src/nnabla/parametric_functions.py:129, :319-485, :563, :946-1117,
:1815, so a network definition written against `PF.*` reads the same here.
Parameters live in a scoped registry like nnabla's (parameter.py:260-355) and
are torch CUDA tensors.
"""
import contextlib
from collections import OrderedDict

import numpy as np
import torch

from . import functions as F

_parameters = OrderedDict()
_scope = []
_device = None


def set_device(device):
    global _device
    _device = torch.device(device)


def _dev():
    return _device if _device is not None else torch.device("cuda", torch.cuda.current_device())


@contextlib.contextmanager
def parameter_scope(name):
    _scope.append(name)
    try:
        yield
    finally:
        _scope.pop()


def get_parameters():
    return _parameters


def clear_parameters():
    _parameters.clear()
    _inq_states.clear()


def get_parameter_or_create(name, shape, initializer):
    """nnabla.parameter.get_parameter_or_create (parameter.py:260): `initializer`
    is a numpy array or a callable shape -> numpy array."""
    key = "/".join(_scope + [name])
    p = _parameters.get(key)
    if p is None:
        a = initializer(shape) if callable(initializer) else np.asarray(initializer)
        a = np.ascontiguousarray(a, dtype=np.float32).reshape(shape)
        p = torch.from_numpy(a).to(_dev())
        _parameters[key] = p
    elif tuple(p.shape) != tuple(shape):
        raise ValueError("parameter %s exists with shape %s, requested %s" % (key, tuple(p.shape), tuple(shape)))
    return p


def _glorot_uniform(inmaps, outmaps, kernel, rng):
    # calc_uniform_lim_glorot (python/src/nnabla/initializer.py:409): b = sqrt(6 / (K (N + M)))
    lim = np.sqrt(6.0 / (np.prod(kernel) * (inmaps + outmaps)))
    return lambda shape: rng.uniform(-lim, lim, size=shape)


def _zeros(shape):
    return np.zeros(shape, np.float32)


def _rng(rng):
    return rng if rng is not None else np.random.RandomState(313)


def affine(inp, n_outmaps, base_axis=1, w_init=None, b_init=None, fix_parameters=False, rng=None, with_bias=True):
    n_outmaps = (n_outmaps,) if isinstance(n_outmaps, int) else tuple(n_outmaps)
    inmaps = int(np.prod(inp.shape[base_axis:]))
    with parameter_scope("affine"):
        w = get_parameter_or_create("W", (inmaps,) + n_outmaps,
                                    w_init or _glorot_uniform(inmaps, int(np.prod(n_outmaps)), (1, 1), _rng(rng)))
        b = get_parameter_or_create("b", n_outmaps, b_init or _zeros) if with_bias else None
    return F.affine(inp, w, b, base_axis)


def binary_weight_affine(inp, n_outmaps, base_axis=1, quantize_zero_to=1.0, w_init=None, wb_init=None, b_init=None,
                         fix_parameters=False, rng=None, with_bias=True):
    n_outmaps = (n_outmaps,) if isinstance(n_outmaps, int) else tuple(n_outmaps)
    inmaps = int(np.prod(inp.shape[base_axis:]))
    init = _glorot_uniform(inmaps, int(np.prod(n_outmaps)), (1, 1), _rng(rng))
    with parameter_scope("bwn_affine"):
        w = get_parameter_or_create("W", (inmaps,) + n_outmaps, w_init or init)
        wb = get_parameter_or_create("Wb", (inmaps,) + n_outmaps, wb_init or init)
        alpha = get_parameter_or_create("alpha", n_outmaps, _zeros)
        b = get_parameter_or_create("b", n_outmaps, b_init or _zeros) if with_bias else None
    return F.binary_weight_affine(inp, w, wb, alpha, b, base_axis, quantize_zero_to)


def binary_connect_affine(inp, n_outmaps, base_axis=1, quantize_zero_to=1.0, w_init=None, wb_init=None, b_init=None,
                          fix_parameters=False, rng=None, with_bias=True):
    n_outmaps = (n_outmaps,) if isinstance(n_outmaps, int) else tuple(n_outmaps)
    inmaps = int(np.prod(inp.shape[base_axis:]))
    init = _glorot_uniform(inmaps, int(np.prod(n_outmaps)), (1, 1), _rng(rng))
    with parameter_scope("bicon_affine"):
        w = get_parameter_or_create("W", (inmaps,) + n_outmaps, w_init or init)
        wb = get_parameter_or_create("Wb", (inmaps,) + n_outmaps, wb_init or init)
        b = get_parameter_or_create("b", n_outmaps, b_init or _zeros) if with_bias else None
    return F.binary_connect_affine(inp, w, wb, b, base_axis, quantize_zero_to)


def convolution(inp, outmaps, kernel, pad=None, stride=None, dilation=None, group=1, channel_last=False,
                w_init=None, b_init=None, base_axis=1, fix_parameters=False, rng=None, with_bias=True):
    inmaps = int(inp.shape[base_axis])
    with parameter_scope("conv"):
        w = get_parameter_or_create("W", (outmaps, inmaps // group) + tuple(kernel),
                                    w_init or _glorot_uniform(inmaps, outmaps, tuple(kernel), _rng(rng)))
        b = get_parameter_or_create("b", (outmaps,), b_init or _zeros) if with_bias else None
    return F.convolution(inp, w, b, base_axis, pad, stride, dilation, group, channel_last)


def binary_weight_convolution(inp, outmaps, kernel, pad=None, stride=None, dilation=None, group=1,
                              quantize_zero_to=1.0, w_init=None, wb_init=None, b_init=None, base_axis=1,
                              fix_parameters=False, rng=None, with_bias=True):
    inmaps = int(inp.shape[base_axis])
    init = _glorot_uniform(inmaps, outmaps, tuple(kernel), _rng(rng))
    shape = (outmaps, inmaps // group) + tuple(kernel)
    with parameter_scope("bwn_conv"):
        w = get_parameter_or_create("W", shape, w_init or init)
        wb = get_parameter_or_create("Wb", shape, wb_init or init)
        alpha = get_parameter_or_create("alpha", (outmaps,), _zeros)
        b = get_parameter_or_create("b", (outmaps,), b_init or _zeros) if with_bias else None
    return F.binary_weight_convolution(inp, w, wb, alpha, b, base_axis, pad, stride, dilation, group,
                                       quantize_zero_to)


def binary_connect_convolution(inp, outmaps, kernel, pad=None, stride=None, dilation=None, group=1,
                               quantize_zero_to=1.0, w_init=None, wb_init=None, b_init=None, base_axis=1,
                               fix_parameters=False, rng=None, with_bias=True):
    inmaps = int(inp.shape[base_axis])
    init = _glorot_uniform(inmaps, outmaps, tuple(kernel), _rng(rng))
    shape = (outmaps, inmaps // group) + tuple(kernel)
    with parameter_scope("bicon_conv"):
        w = get_parameter_or_create("W", shape, w_init or init)
        wb = get_parameter_or_create("Wb", shape, wb_init or init)
        b = get_parameter_or_create("b", (outmaps,), b_init or _zeros) if with_bias else None
    return F.binary_connect_convolution(inp, w, wb, b, base_axis, pad, stride, dilation, group, quantize_zero_to)


def batch_normalization(inp, axes=[1], decay_rate=0.9, eps=1e-5, batch_stat=True, output_stat=False,
                        fix_parameters=False, param_init=None, no_scale=False, no_bias=False):
    ax = axes[0]
    shape = [1] * inp.dim()
    shape[ax] = int(inp.shape[ax])
    shape = tuple(shape)
    init = param_init or {}
    with parameter_scope("bn"):
        beta = None if no_bias else get_parameter_or_create("beta", shape, init.get("beta", _zeros))
        gamma = None if no_scale else get_parameter_or_create(
            "gamma", shape, init.get("gamma", lambda s: np.ones(s, np.float32)))
        mean = get_parameter_or_create("mean", shape, init.get("mean", _zeros))
        var = get_parameter_or_create("var", shape, init.get("var", lambda s: np.ones(s, np.float32)))
    return F.batch_normalization(inp, beta, gamma, mean, var, axes, decay_rate, eps, batch_stat, output_stat)


def fixed_point_quantized_affine(inp, n_outmaps, base_axis=1, w_init=None, b_init=None, fix_parameters=False, rng=None,
                                 with_bias=True, quantize_w=True, sign_w=True, n_w=8, delta_w=2 ** -4,
                                 ste_fine_grained_w=True, quantize_b=True, sign_b=True, n_b=8, delta_b=2 ** -4,
                                 ste_fine_grained_b=True, input_delta=None):
    """Fixed-Point Quantized Affine (python/src/nnabla/parametric_functions.py:2296-2408):
    y = x . Q(W) + Q(b), with the quantized copies kept as parameters W_q / b_q.
    input_delta=d declares that inp holds multiples of d with at most 8 bits
    (the output of fixed_point_quantize); with 8-bit weights the product then
    runs on the exact int8 tensor-core path."""
    n_outmaps = (n_outmaps,) if isinstance(n_outmaps, int) else tuple(n_outmaps)
    inmaps = int(np.prod(inp.shape[base_axis:]))
    with parameter_scope("fp_quantized_affine"):
        w = get_parameter_or_create("W", (inmaps,) + n_outmaps,
                                    w_init or _glorot_uniform(inmaps, int(np.prod(n_outmaps)), (1, 1), _rng(rng)))
        real_w = w
        if quantize_w:
            w_q = get_parameter_or_create("W_q", (inmaps,) + n_outmaps, _zeros)
            real_w = F.fixed_point_quantize(w, sign_w, n_w, delta_w, True, ste_fine_grained_w, outputs=[w_q])
        real_b = None
        if with_bias:
            b = get_parameter_or_create("b", n_outmaps, b_init or _zeros)
            real_b = b
            if quantize_b:
                b_q = get_parameter_or_create("b_q", n_outmaps, _zeros)
                real_b = F.fixed_point_quantize(b, sign_b, n_b, delta_b, True, ste_fine_grained_b, outputs=[b_q])
    exact = input_delta is not None and quantize_w and (n_w - (1 if sign_w else 0)) <= 7
    return F.affine(inp, real_w, real_b, base_axis, fixed_point=(input_delta, delta_w) if exact else None)


def fixed_point_quantized_convolution(inp, outmaps, kernel, pad=None, stride=None, dilation=None, group=1,
                                      channel_last=False, w_init=None, b_init=None, base_axis=1, fix_parameters=False,
                                      rng=None, with_bias=True, quantize_w=True, sign_w=True, n_w=8, delta_w=2 ** -4,
                                      ste_fine_grained_w=True, quantize_b=True, sign_b=True, n_b=8, delta_b=2 ** -4,
                                      ste_fine_grained_b=True, input_delta=None):
    """Fixed-Point Quantized Convolution (python/src/nnabla/parametric_functions.py:2411-2530).
    With input_delta and 8-bit weights the convolution is the exact int8 one;
    without them only few-channel inputs are supported (the full-precision stem kernel)."""
    inmaps = int(inp.shape[base_axis])
    with parameter_scope("fp_quantized_conv"):
        w = get_parameter_or_create("W", (outmaps, inmaps // group) + tuple(kernel),
                                    w_init or _glorot_uniform(inmaps, outmaps, tuple(kernel), _rng(rng)))
        real_w = w
        if quantize_w:
            w_q = get_parameter_or_create("W_q", (outmaps, inmaps // group) + tuple(kernel), _zeros)
            real_w = F.fixed_point_quantize(w, sign_w, n_w, delta_w, True, ste_fine_grained_w, outputs=[w_q])
        real_b = None
        if with_bias:
            b = get_parameter_or_create("b", (outmaps,), b_init or _zeros)
            real_b = b
            if quantize_b:
                b_q = get_parameter_or_create("b_q", (outmaps,), _zeros)
                real_b = F.fixed_point_quantize(b, sign_b, n_b, delta_b, True, ste_fine_grained_b, outputs=[b_q])
    exact = input_delta is not None and quantize_w and (n_w - (1 if sign_w else 0)) <= 7
    return F.convolution(inp, real_w, real_b, base_axis, pad, stride, dilation, group, channel_last,
                         fixed_point=(input_delta, delta_w) if exact else None)


def pow2_quantized_affine(inp, n_outmaps, base_axis=1, w_init=None, b_init=None, fix_parameters=False, rng=None,
                          with_bias=True, quantize_w=True, sign_w=True, with_zero_w=False, n_w=8, m_w=2,
                          ste_fine_grained_w=True, quantize_b=True, sign_b=True, with_zero_b=False, n_b=8, m_b=2,
                          ste_fine_grained_b=True):
    """Pow2 Quantized Affine (python/src/nnabla/parametric_functions.py:2533-2645)."""
    n_outmaps = (n_outmaps,) if isinstance(n_outmaps, int) else tuple(n_outmaps)
    inmaps = int(np.prod(inp.shape[base_axis:]))
    with parameter_scope("pow2_quantized_affine"):
        w = get_parameter_or_create("W", (inmaps,) + n_outmaps,
                                    w_init or _glorot_uniform(inmaps, int(np.prod(n_outmaps)), (1, 1), _rng(rng)))
        real_w = w
        if quantize_w:
            w_q = get_parameter_or_create("W_q", (inmaps,) + n_outmaps, _zeros)
            real_w = F.pow2_quantize(w, sign_w, with_zero_w, n_w, m_w, True, ste_fine_grained_w, outputs=[w_q])
        real_b = None
        if with_bias:
            b = get_parameter_or_create("b", n_outmaps, b_init or _zeros)
            real_b = b
            if quantize_b:
                b_q = get_parameter_or_create("b_q", n_outmaps, _zeros)
                real_b = F.pow2_quantize(b, sign_b, with_zero_b, n_b, m_b, True, ste_fine_grained_b, outputs=[b_q])
    return F.affine(inp, real_w, real_b, base_axis)


def pruned_affine(inp, n_outmaps, base_axis=1, w_init=None, b_init=None, fix_parameters=False, rng=None,
                  with_bias=True, prune_w=True, rate_w=0.9, prune_b=True, rate_b=0.9):
    """Pruned Affine (python/src/nnabla/parametric_functions.py:2765-2864)."""
    n_outmaps = (n_outmaps,) if isinstance(n_outmaps, int) else tuple(n_outmaps)
    inmaps = int(np.prod(inp.shape[base_axis:]))
    with parameter_scope("pruned_affine"):
        w = get_parameter_or_create("W", (inmaps,) + n_outmaps,
                                    w_init or _glorot_uniform(inmaps, int(np.prod(n_outmaps)), (1, 1), _rng(rng)))
        real_w = w
        if prune_w:
            w_q = get_parameter_or_create("W_q", (inmaps,) + n_outmaps, _zeros)
            real_w = F.prune(w, rate_w, outputs=[w_q])
        real_b = None
        if with_bias:
            b = get_parameter_or_create("b", n_outmaps, b_init or _zeros)
            real_b = b
            if prune_b:
                b_q = get_parameter_or_create("b_q", n_outmaps, _zeros)
                real_b = F.prune(b, rate_b, outputs=[b_q])
    return F.affine(inp, real_w, real_b, base_axis)


_inq_states = {}


def _inq_layer(scope, shape, init, i_init, b_shape, b_init, with_bias, seed):
    """Parameters "W", "I" (indicators: 0 learnable, 1 fixed; int32 here, where nnabla stores them as its
    default float arrays and the function reads them as int) and "b" of an INQ layer, plus the state the
    reference keeps inside the function instance, kept per scope."""
    with parameter_scope(scope):
        w = get_parameter_or_create("W", shape, init)
        key = "/".join(_scope + ["I"])
        ind = _parameters.get(key)
        if ind is None:
            a = np.zeros(shape) if i_init is None else (i_init(shape) if callable(i_init) else np.asarray(i_init))
            ind = torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32).reshape(shape)).to(_dev())
            _parameters[key] = ind
        elif ind.dtype != torch.int32:  # loaded from a parameter file, which holds floats
            ind = _parameters[key] = ind.to(torch.int32).contiguous()
        b = get_parameter_or_create("b", b_shape, b_init if b_init is not None else _zeros) if with_bias else None
        state = _inq_states.get(key)
        if state is None or state.old_weights.shape != w.shape:
            state = _inq_states[key] = F.INQState(w, seed)
    return w, ind, b, state


def inq_affine(inp, n_outmaps, base_axis=1, num_bits=4, inq_iterations=(), selection_algorithm='random', seed=-1,
               w_init=None, i_init=None, b_init=None, fix_parameters=False, rng=None, with_bias=True):
    """python/src/nnabla/parametric_functions.py:493-557 (scope "inq_affine", parameters W, I, b)."""
    n_outmaps = (n_outmaps,) if isinstance(n_outmaps, int) else tuple(n_outmaps)
    inmaps = int(np.prod(inp.shape[base_axis:]))
    init = w_init if w_init is not None else _glorot_uniform(inmaps, int(np.prod(n_outmaps)), (1, 1), _rng(rng))
    w, ind, b, state = _inq_layer("inq_affine", (inmaps,) + n_outmaps, init, i_init, n_outmaps, b_init, with_bias, seed)
    return F.inq_affine(inp, w, ind, b, base_axis, num_bits, inq_iterations, selection_algorithm, seed, state)


def inq_convolution(inp, outmaps, kernel, pad=None, stride=None, dilation=None, group=1, num_bits=4,
                    inq_iterations=(), selection_algorithm='random', seed=-1, w_init=None, i_init=None, b_init=None,
                    base_axis=1, fix_parameters=False, rng=None, with_bias=True):
    """python/src/nnabla/parametric_functions.py:1126-1196 (scope "inq_conv", parameters W, I, b)."""
    inmaps = int(inp.shape[base_axis])
    init = w_init if w_init is not None else _glorot_uniform(inmaps, outmaps, tuple(kernel), _rng(rng))
    shape = (outmaps, inmaps // group) + tuple(kernel)
    w, ind, b, state = _inq_layer("inq_conv", shape, init, i_init, (outmaps,), b_init, with_bias, seed)
    return F.inq_convolution(inp, w, ind, b, base_axis, pad, stride, dilation, group, num_bits, inq_iterations,
                             selection_algorithm, seed, state)


def _constant(value):
    return lambda shape: np.full(shape, value, np.float32)


def min_max_quantize(x, ql_min=0, ql_max=255, decay=0.999, x_min_max=False, ema=False, ste_fine_grained=True,
                     eps=0.01, qr_min_init=None, qr_max_init=None, fix_parameters=False, outputs=None,
                     name="min_max_quantize"):
    """Min-max quantization with its ranges kept as parameters
    (python/src/nnabla/parametric_functions.py:2971-3097): scalar quantization
    levels become (1, ..., 1)-shaped parameters ql_min / ql_max, the ranges
    qr_min / qr_max start at -6 / 6 unless initialisers are given."""
    with parameter_scope(name):
        ones = (1,) * x.dim()
        if isinstance(ql_min, (int, float)):
            ql_min = get_parameter_or_create("ql_min", ones, _constant(ql_min))
        if isinstance(ql_max, (int, float)):
            ql_max = get_parameter_or_create("ql_max", ones, _constant(ql_max))
        shape = tuple(ql_min.shape)
        qr_min = get_parameter_or_create("qr_min", shape, qr_min_init or _constant(-6.0))
        qr_max = get_parameter_or_create("qr_max", shape, qr_max_init or _constant(6.0))
    return F.min_max_quantize(x, qr_min, qr_max, ql_min, ql_max, decay, x_min_max, ema, ste_fine_grained, eps,
                              outputs=outputs)


def min_max_quantized_affine(inp, n_outmaps, base_axis=1, w_init=None, b_init=None, fix_parameters=False, rng=None,
                             with_bias=True, quantize_w=True, ql_min_w=0, ql_max_w=255, w_min_max=False,
                             qr_min_w_init=None, qr_max_w_init=None, ste_fine_grained_w=True, quantize_b=True,
                             ql_min_b=0, ql_max_b=255, b_min_max=False, qr_min_b_init=None, qr_max_b_init=None,
                             ste_fine_grained_b=True, eps=0.01):
    """Min-max Quantized Affine (python/src/nnabla/parametric_functions.py:3110-3256):
    weight ranges start at -2 / 2, bias ranges at -6 / 6."""
    n_outmaps = (n_outmaps,) if isinstance(n_outmaps, int) else tuple(n_outmaps)
    inmaps = int(np.prod(inp.shape[base_axis:]))
    with parameter_scope("min_max_quantized_affine"):
        w = get_parameter_or_create("W", (inmaps,) + n_outmaps,
                                    w_init or _glorot_uniform(inmaps, int(np.prod(n_outmaps)), (1, 1), _rng(rng)))
        real_w = w
        if quantize_w:
            w_q = get_parameter_or_create("W_q", (inmaps,) + n_outmaps, _zeros)
            real_w = min_max_quantize(w, ql_min_w, ql_max_w, 0.999, w_min_max, False, ste_fine_grained_w, eps,
                                      qr_min_w_init or _constant(-2.0), qr_max_w_init or _constant(2.0),
                                      fix_parameters, outputs=[w_q], name="min_max_quantize_w")
        real_b = None
        if with_bias:
            b = get_parameter_or_create("b", n_outmaps, b_init or _zeros)
            real_b = b
            if quantize_b:
                b_q = get_parameter_or_create("b_q", n_outmaps, _zeros)
                real_b = min_max_quantize(b, ql_min_b, ql_max_b, 0.999, b_min_max, False, ste_fine_grained_b, eps,
                                          qr_min_b_init or _constant(-6.0), qr_max_b_init or _constant(6.0),
                                          fix_parameters, outputs=[b_q], name="min_max_quantize_b")
    return F.affine(inp, real_w, real_b, base_axis)


# ---------------------------------------------------------------------------
# Parameter files in nnabla's `.protobuf` format, so that the parameters of a network trained or converted
# here ("W", the binarised "Wb" and "alpha", BatchNormalization statistics, INQ indicators) load in nnabla
# with nn.load_parameters and the other way round. Written by hand on the wire format (no generated module):
#   NNablaProtoBuf { repeated Parameter parameter = 200; }
#   Parameter { string variable_name = 1; Shape shape = 20; repeated float data = 100; bool need_grad = 101; }
#   Shape { repeated int64 dim = 1 [packed]; }
# (src/nbla/proto/nnabla.proto.tmpl:24-26, :38-49, :105-110; the writer of
# python/src/nnabla/utils/get_file_handle.py:476-486, the reader of python/src/nnabla/parameter.py:392-399.)
# ---------------------------------------------------------------------------
_NO_GRAD_NAMES = ("Wb", "alpha", "mean", "var", "I")  # registered with need_grad=False by nnabla's layers


def _varint(n):
    n &= (1 << 64) - 1
    out = bytearray()
    while True:
        b = n & 0x7F
        n >>= 7
        if n:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _field(number, wire_type, payload):
    head = _varint((number << 3) | wire_type)
    return head + (_varint(len(payload)) + payload if wire_type == 2 else payload)


def _read_varint(buf, pos):
    shift = value = 0
    while True:
        if pos >= len(buf):
            raise ValueError("truncated varint")
        b = buf[pos]
        pos += 1
        value |= (b & 0x7F) << shift
        if not b & 0x80:
            return value, pos
        shift += 7
        if shift > 63:
            raise ValueError("varint too long")


def _fields(buf):
    """(field number, wire type, value) of one message; value is an int (varint, fixed) or a memoryview."""
    pos = 0
    view = memoryview(buf)
    while pos < len(buf):
        key, pos = _read_varint(buf, pos)
        number, wt = key >> 3, key & 7
        if wt == 0:
            value, pos = _read_varint(buf, pos)
        elif wt == 1:
            value, pos = int.from_bytes(buf[pos:pos + 8], "little"), pos + 8
        elif wt == 5:
            value, pos = int.from_bytes(buf[pos:pos + 4], "little"), pos + 4
        elif wt == 2:
            n, pos = _read_varint(buf, pos)
            if pos + n > len(buf):
                raise ValueError("truncated field")
            value, pos = view[pos:pos + n], pos + n
        else:
            raise ValueError("unsupported wire type %d" % wt)
        yield number, wt, value


def save_parameters(path, params=None):
    """nn.save_parameters for the `.protobuf` format (python/src/nnabla/parameter.py:424-447)."""
    if not str(path).endswith(".protobuf"):
        raise ValueError("Only supported .protobuf.")
    params = get_parameters() if params is None else params
    out = bytearray()
    for name, p in params.items():
        a = np.asarray(p.detach().cpu().numpy() if isinstance(p, torch.Tensor) else p)
        shape = b"".join(_varint(int(d)) for d in a.shape)
        msg = _field(1, 2, name.encode("utf-8"))
        msg += _field(20, 2, _field(1, 2, shape) if a.ndim else b"")
        msg += _field(100, 2, a.astype("<f4").tobytes())
        if name.rsplit("/", 1)[-1] not in _NO_GRAD_NAMES:
            msg += _field(101, 0, _varint(1))
        out += _field(200, 2, msg)
    with open(path, "wb") as f:
        f.write(bytes(out))


def load_parameters(path):
    """nn.load_parameters for the `.protobuf` format: every Parameter of the file replaces or creates the
    entry of that name in the registry (set_parameter_from_proto, parameter.py:392-399). Returns
    {name: need_grad}."""
    if not str(path).endswith(".protobuf"):
        raise ValueError("Only supported .protobuf.")
    with open(path, "rb") as f:
        buf = f.read()
    flags = OrderedDict()
    for number, wt, value in _fields(buf):
        if number != 200 or wt != 2:
            continue  # networks, optimizers, ... of a full model file are not parameters
        name, dims, chunks, need_grad = "", [], [], False
        for n2, w2, v2 in _fields(bytes(value)):
            if n2 == 1 and w2 == 2:
                name = bytes(v2).decode("utf-8")
            elif n2 == 20 and w2 == 2:
                for n3, w3, v3 in _fields(bytes(v2)):
                    if n3 == 1 and w3 == 2:  # packed
                        b3, pos = bytes(v3), 0
                        while pos < len(b3):
                            d, pos = _read_varint(b3, pos)
                            dims.append(d)
                    elif n3 == 1 and w3 == 0:
                        dims.append(v3)
            elif n2 == 100 and w2 == 2:  # packed floats
                chunks.append(np.frombuffer(bytes(v2), dtype="<f4"))
            elif n2 == 100 and w2 == 5:  # one float per field
                chunks.append(np.array([v2], dtype="<u4").view("<f4"))
            elif n2 == 101 and w2 == 0:
                need_grad = bool(v2)
        data = np.concatenate(chunks) if chunks else np.zeros(0, np.float32)
        if data.size != int(np.prod(dims, dtype=np.int64)):
            raise ValueError("parameter %s: %d values for shape %s" % (name, data.size, tuple(dims)))
        _parameters[name] = torch.from_numpy(data.astype(np.float32).reshape(dims)).to(_dev())
        flags[name] = need_grad
    return flags
