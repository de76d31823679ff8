"""The nnabla extension backend "b200:float" against nnabla's own "cpu:float"
context in the same process: the function is created through nnabla's
registry, fed through nnabla Variables / SyncedArrays (device arrays, caching
allocator and synchronizers of the extension), and only the context differs.
Quantizer outputs, signs and the companions must match bit for bit; alpha to
fp32 summation error; contraction outputs within 1e-5 of the output RMS."""
import numpy as np
import pytest

import cases
import ext_harness as H
from golden_util import bits

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not H.available(), reason="extension library not built")]
CPU, B200 = "cpu:float", "b200:float"


@pytest.fixture(scope="module", autouse=True)
def _init():
    H.init()


def both(op, scalars, ivecs, inputs, n_out=1, prequant=None):
    c = H.forward(CPU, op, scalars, ivecs, inputs, n_out, prequant)
    g = H.forward(B200, op, scalars, ivecs, inputs, n_out, prequant)
    assert c[2] == g[2] == op  # name() is the reference's
    return c, g


@pytest.mark.parametrize("sign,n,delta", cases.FXP_GRID)
def test_fixed_point_quantize(sign, n, delta):
    n_eff = n - 1 if sign else n
    x = np.concatenate([cases.fxp_input().ravel(), cases.edge_values_fxp(np.float32(delta), n_eff)])
    c, g = both("FixedPointQuantize", [sign, n, delta, True], [], [x])
    assert np.array_equal(bits(g[0][0]), bits(c[0][0]))


@pytest.mark.parametrize("sign,with_zero,n,m", cases.POW2_GRID + [(True, True, 8, 1)])
def test_pow2_quantize(sign, with_zero, n, m):
    x = np.concatenate([cases.fxp_input().ravel(), cases.edge_values_pow2()])
    c, g = both("Pow2Quantize", [sign, with_zero, n, m, True], [], [x])
    assert np.array_equal(bits(g[0][0]), bits(c[0][0]))


@pytest.mark.parametrize("shapes,decay,x_min_max,ema", cases.MINMAX_GRID)
def test_min_max_quantize(shapes, decay, x_min_max, ema):
    ins = list(cases.minmax_inputs(*shapes))
    c, g = both("MinMaxQuantize", [decay, x_min_max, ema, True, 0.01], [], ins)
    assert np.array_equal(bits(g[0][0]), bits(c[0][0]))
    assert np.array_equal(bits(g[1][1]), bits(c[1][1]))  # qr_min written back
    assert np.array_equal(bits(g[1][2]), bits(c[1][2]))  # qr_max written back


@pytest.mark.parametrize("xs,ws,base_axis", cases.AFFINE_CASES)
@pytest.mark.parametrize("qzt", cases.QZT)
def test_binary_affines(xs, ws, base_axis, qzt):
    x, w, b = cases.affine_inputs(xs, ws, with_zeros=True)
    wb = np.zeros_like(w)
    alpha = np.zeros(int(np.prod(ws[1:])), np.float32)
    c, g = both("BinaryWeightAffine", [base_axis, qzt], [], [x, w, wb, alpha, b])
    assert np.array_equal(bits(g[1][2]), bits(c[1][2]))                      # Wb
    np.testing.assert_allclose(g[1][3], c[1][3], rtol=2e-6)                  # alpha
    assert g[0][0].shape == c[0][0].shape and cases.rel_rms(g[0][0], c[0][0]) < 1e-5
    c, g = both("BinaryConnectAffine", [base_axis, qzt], [], [x, w, wb, b])
    assert np.array_equal(bits(g[1][2]), bits(c[1][2]))
    assert cases.rel_rms(g[0][0], c[0][0]) < 1e-5


@pytest.mark.parametrize("xs,ws,pad,stride,dilation,group", cases.CONV_CASES)
def test_binary_convolutions(xs, ws, pad, stride, dilation, group):
    x, w, b = cases.conv_inputs(xs, ws, with_zeros=True)
    wb, alpha = np.zeros_like(w), np.zeros(ws[0], np.float32)
    c, g = both("BinaryWeightConvolution", [1, group, 1.0], [pad, stride, dilation], [x, w, wb, alpha, b])
    assert np.array_equal(bits(g[1][2]), bits(c[1][2]))
    np.testing.assert_allclose(g[1][3], c[1][3], rtol=2e-6)
    assert g[0][0].shape == c[0][0].shape and cases.rel_rms(g[0][0], c[0][0]) < 1e-5
    c, g = both("BinaryConnectConvolution", [1, group, 1.0], [pad, stride, dilation], [x, w, wb, b])
    assert np.array_equal(bits(g[1][2]), bits(c[1][2]))
    assert cases.rel_rms(g[0][0], c[0][0]) < 1e-5


def test_fixed_point_tag_selects_the_exact_int8_paths():
    """FixedPointQuantize -> Affine / BinaryWeightConvolution inside nnabla's
    machinery: the extension recognises the quantizer's output array and runs
    the int8 contraction; the fixed-point affine then equals the CPU result
    bit for bit."""
    rng = np.random.RandomState(0)
    x = rng.randn(96, 256).astype(np.float32)
    w = (0.02 * rng.randn(256, 320)).astype(np.float32)
    b = (0.01 * rng.randn(320)).astype(np.float32)
    c, g = both("Affine", [1], [], [x, w, b], prequant=[2.0 ** -5, 2.0 ** -10, 0])
    assert np.array_equal(bits(g[0][0]), bits(c[0][0]))
    xc = np.maximum(rng.randn(2, 64, 14, 14), 0).astype(np.float32)
    wc = (rng.randn(64, 64, 3, 3) * np.sqrt(2.0 / 576)).astype(np.float32)
    wb, alpha = np.zeros_like(wc), np.zeros(64, np.float32)
    c, g = both("BinaryWeightConvolution", [1, 1, 1.0], [(1, 1), (1, 1), (1, 1)], [xc, wc, wb, alpha],
                prequant=[2.0 ** -4, 0, 0, 0])
    assert cases.rel_rms(g[0][0], c[0][0]) < 2e-6


def test_companions_and_full_precision_layers():
    rng = np.random.RandomState(cases.SEED)
    x = rng.randn(2, 6, 9, 12).astype(np.float32)
    beta, gamma, mean = (rng.randn(1, 6, 1, 1).astype(np.float32) for _ in range(3))
    var = (rng.rand(1, 6, 1, 1) + 0.1).astype(np.float32)
    c, g = both("BatchNormalization", [0.9, 1e-5, False, False, False], [(1,)], [x, beta, gamma, mean, var])
    assert np.array_equal(bits(g[0][0]), bits(c[0][0]))
    for op, sc, iv, ins in [("ReLU", [False], [], [x]), ("Add2", [False], [], [x, x[::-1].copy()]),
                            ("MaxPooling", [True, False], [(3, 3), (2, 2), (1, 1)], [x]),
                            ("GlobalAveragePooling", [], [], [x])]:
        c, g = both(op, sc, iv, ins)
        assert np.array_equal(bits(g[0][0]), bits(c[0][0])), op
    xs = rng.randn(2, 3, 20, 20).astype(np.float32)
    ws = rng.randn(8, 3, 7, 7).astype(np.float32)
    c, g = both("Convolution", [1, 1, False], [(3, 3), (2, 2), (1, 1)], [xs, ws])
    assert cases.rel_rms(g[0][0], c[0][0]) < 1e-6
    xa, wa, ba = cases.affine_inputs((3, 5, 7), (35, 40))
    c, g = both("Affine", [1], [], [xa, wa, ba])
    assert cases.rel_rms(g[0][0], c[0][0]) < 1e-5


def test_companions_training_side():
    """Batch-statistics BatchNormalization and the backward passes of the companions through
    Function::forward / Function::backward of both backends."""
    rng = np.random.RandomState(cases.SEED + 1)
    x = (rng.randn(4, 6, 9, 12) * 2 + 0.5).astype(np.float32)
    x[rng.rand(*x.shape) < 0.1] = 0.0
    beta, gamma, mean = (rng.randn(1, 6, 1, 1).astype(np.float32) for _ in range(3))
    var = (rng.rand(1, 6, 1, 1) + 0.5).astype(np.float32)
    bn_in = [x, beta, gamma, mean, var]
    # forward with batch statistics: y, batch mean, batch variance; the running statistics are written in place
    c, g = both("BatchNormalization", [0.9, 1e-5, True, False, False], [(1,)], bn_in, n_out=3)
    for k in range(3):
        assert np.allclose(g[0][k], c[0][k], rtol=1e-4, atol=1e-5), k
    for k in (3, 4):
        assert np.allclose(g[1][k], c[1][k], rtol=1e-4, atol=1e-5), k
    dy, dx0 = cases.grad_inputs(x)
    small = lambda: rng.randn(1, 6, 1, 1).astype(np.float32)
    for batch_stat in (True, False):
        for accum in (False, True):
            ogs = [dy] + ([small(), small()] if batch_stat else [])
            g0 = [dx0, small(), small(), small(), small()]
            args = ("BatchNormalization", [0.9, 1e-5, batch_stat, False, False], [(1,)], bn_in, ogs,
                    [True, True, True, False, False], [accum] * 3 + [False, False], g0)
            cb, gb = H.backward(CPU, *args), H.backward(B200, *args)
            for k in range(3):
                tol = 2e-5 * (np.abs(cb[0][k]).max() + 1.0) * (1 if k == 0 else 30)
                assert np.abs(gb[0][k] - cb[0][k]).max() <= tol, (batch_stat, accum, k)
    for op, sc, iv, ins, exact in [("ReLU", [False], [], [x], True), ("Add2", [False], [], [x, x[::-1].copy()], True),
                                   ("MaxPooling", [True, False], [(3, 3), (2, 2), (1, 1)], [x], True),
                                   ("GlobalAveragePooling", [], [], [x], True)]:
        yshape = H.forward(CPU, op, sc, iv, ins)[0][0].shape
        gy = rng.randn(*yshape).astype(np.float32)
        for accum in (False, True):
            g0 = [rng.randn(*a.shape).astype(np.float32) for a in ins]
            args = (op, sc, iv, ins, [gy], [True] * len(ins), [accum] * len(ins), g0)
            cb, gb = H.backward(CPU, *args), H.backward(B200, *args)
            for k in range(len(ins)):
                assert np.array_equal(bits(gb[0][k]), bits(cb[0][k])), (op, accum, k)
    # full-precision convolution: input, weight and bias gradients
    xs = rng.randn(2, 3, 20, 20).astype(np.float32)
    ws = rng.randn(8, 3, 7, 7).astype(np.float32)
    bs = rng.randn(8).astype(np.float32)
    gy = rng.randn(2, 8, 10, 10).astype(np.float32)
    g0 = [rng.randn(*xs.shape).astype(np.float32), rng.randn(*ws.shape).astype(np.float32),
          rng.randn(8).astype(np.float32)]
    for accum in (True, False):
        args = ("Convolution", [1, 1, False], [(3, 3), (2, 2), (1, 1)], [xs, ws, bs], [gy], [True, True, True],
                [accum] * 3, g0)
        cb, gb = H.backward(CPU, *args), H.backward(B200, *args)
        for k in range(3):
            assert cases.rel_rms(gb[0][k], cb[0][k]) < 1e-5, (accum, k)


def test_half_type_config_resolves_to_the_float_implementations():
    """Context(['b200:half', 'b200:float']) (what an nnabla extension hands out for type_config='half'): nothing is
    registered under 'b200:half', so nnabla's registry goes on to 'b200:float' (function_registry.hpp:57-72)."""
    x = cases.fxp_input()
    g = H.forward(B200, "FixedPointQuantize", [True, 8, 2.0 ** -4, True], [], [x])
    h = H.forward("b200:half", "FixedPointQuantize", [True, 8, 2.0 ** -4, True], [], [x])
    assert h[2] == "FixedPointQuantize" and np.array_equal(bits(h[0][0]), bits(g[0][0]))
    xa, wa, ba = cases.affine_inputs((3, 5, 7), (35, 40))
    wb, al = np.zeros_like(wa), np.zeros(wa.shape[1], np.float32)
    g = H.forward(B200, "BinaryWeightAffine", [1, 1.0], [], [xa, wa, wb, al, ba])
    h = H.forward("b200:half", "BinaryWeightAffine", [1, 1.0], [], [xa, wa, wb, al, ba])
    assert np.array_equal(bits(h[0][0]), bits(g[0][0]))


def test_errors_surface_as_exceptions():
    x = np.zeros((4, 8), np.float32)
    with pytest.raises(RuntimeError, match="positive"):
        H.forward(B200, "FixedPointQuantize", [True, 0, 0.5, True], [], [x])
    w = np.zeros((9, 3), np.float32)
    with pytest.raises(RuntimeError, match="mismatch"):
        H.forward(B200, "BinaryWeightAffine", [1, 1.0], [], [x, w, w.copy(), np.zeros(3, np.float32)])
    with pytest.raises(RuntimeError, match="not implemented|not_implemented|not supported"):
        H.forward(B200, "BatchNormalization", [0.9, 1e-5, True, False, False], [(1, 2)],
                  [x.reshape(4, 8, 1, 1)] + [np.zeros((1, 8, 1, 1), np.float32)] * 4)


# ---- backward passes of the quantizers through Function::backward -----------

def both_backward(op, scalars, inputs, dy, pd, ac, g0):
    c = H.backward(CPU, op, scalars, [], inputs, [dy], pd, ac, g0)
    g = H.backward(B200, op, scalars, [], inputs, [dy], pd, ac, g0)
    return c, g


@pytest.mark.parametrize("sign,n,delta", cases.FXP_GRID[:4])
@pytest.mark.parametrize("fine", [True, False])
@pytest.mark.parametrize("accum", [False, True])
def test_fixed_point_quantize_backward(sign, n, delta, fine, accum):
    x = cases.fxp_backward_input(delta, n - 1 if sign else n)
    dy, dx0 = cases.grad_inputs(x)
    c, g = both_backward("FixedPointQuantize", [sign, n, delta, fine], [x], dy, [True], [accum], [dx0])
    assert np.array_equal(bits(g[0][0]), bits(c[0][0]))


@pytest.mark.parametrize("sign,with_zero,n,m", cases.POW2_GRID[::3] + [(True, True, 8, 1)])
@pytest.mark.parametrize("fine", [True, False])
@pytest.mark.parametrize("accum", [False, True])
def test_pow2_quantize_backward(sign, with_zero, n, m, fine, accum):
    x = cases.pow2_backward_input(m)
    dy, dx0 = cases.grad_inputs(x)
    c, g = both_backward("Pow2Quantize", [sign, with_zero, n, m, fine], [x], dy, [True], [accum], [dx0])
    assert np.array_equal(bits(g[0][0]), bits(c[0][0]))


@pytest.mark.parametrize("shapes,decay,x_min_max,ema", cases.MINMAX_GRID[::2])
@pytest.mark.parametrize("fine", [True, False])
@pytest.mark.parametrize("accum", [False, True])
def test_min_max_quantize_backward(shapes, decay, x_min_max, ema, fine, accum):
    ins = list(cases.minmax_inputs(*shapes))
    dy, dx0 = cases.grad_inputs(ins[0])
    rng = np.random.RandomState(3)
    g0 = [dx0] + [rng.randn(*ins[1].shape).astype(np.float32) for _ in range(4)]
    ranges = not (x_min_max or ema)
    pd = [True, ranges, ranges, False, False]
    c, g = both_backward("MinMaxQuantize", [decay, x_min_max, ema, fine, 0.01], ins, dy, pd, [accum] * 5, g0)
    assert np.array_equal(bits(g[0][0]), bits(c[0][0]))
    per_q = ins[0].size // ins[1].size
    tol = 1e-6 * per_q ** 0.5 * (np.abs(dy).max() + 1)
    for k in (1, 2):
        if ranges:
            assert np.allclose(g[0][k], c[0][k], rtol=1e-5, atol=tol)
        else:
            assert np.array_equal(bits(g[0][k]), bits(c[0][k]))


@pytest.mark.parametrize("xs,ws,base_axis", cases.AFFINE_CASES)
@pytest.mark.parametrize("accum", [False, True])
def test_affine_family_backward(xs, ws, base_axis, accum):
    x, w, b = cases.affine_inputs(xs, ws, with_zeros=True)
    rng = np.random.RandomState(1)
    dy = rng.randn(*(tuple(xs[:base_axis]) + tuple(ws[1:]))).astype(np.float32)
    gx, gw, gb = (rng.randn(*s).astype(np.float32) for s in (xs, ws, ws[1:]))
    wb, alpha = np.zeros_like(w), np.zeros(int(np.prod(ws[1:])), np.float32)
    runs = [
        ("Affine", [base_axis], [x, w, b], [True, True, True], [gx, gw, gb]),
        ("BinaryWeightAffine", [base_axis, 1.0], [x, w, wb, alpha, b], [True, True, False, False, True],
         [gx, gw, wb, alpha, gb]),
        ("BinaryConnectAffine", [base_axis, 0.0], [x, w, wb, b], [True, True, False, True], [gx, gw, wb, gb]),
    ]
    for op, scalars, ins, pd, g0 in runs:
        c = H.backward(CPU, op, scalars, [], ins, [dy], pd, [accum] * len(ins), g0)
        g = H.backward(B200, op, scalars, [], ins, [dy], pd, [accum] * len(ins), g0)
        for i, p in enumerate(pd):
            # (the reference leaves the weight gradient in the BINARY weights' gradient too, binary_connect_affine.cpp:77-92)
            if p or (op == "BinaryConnectAffine" and i == 2):
                assert cases.rel_rms(g[0][i], c[0][i]) < 1e-5, (op, i)
            else:
                assert np.array_equal(bits(g[0][i]), bits(c[0][i])), (op, i)


@pytest.mark.parametrize("xs,ws,pad,stride,dil,grp", cases.CONV_CASES)
@pytest.mark.parametrize("accum", [False, True])
def test_binary_convolutions_backward(xs, ws, pad, stride, dil, grp, accum):
    from oracle import oracle
    x, w, b = cases.conv_inputs(xs, ws, with_zeros=True)
    rng = np.random.RandomState(2)
    dy = rng.randn(*oracle.conv_out_shape(xs, ws, pad, stride, dil)).astype(np.float32)
    gx, gw, gb = (rng.randn(*s).astype(np.float32) for s in (xs, ws, (ws[0],)))
    wb, alpha = np.zeros_like(w), np.zeros(ws[0], np.float32)
    runs = [
        ("BinaryWeightConvolution", [1, grp, 1.0], [x, w, wb, alpha, b], [True, True, False, False, True],
         [gx, gw, wb, alpha, gb]),
        ("BinaryConnectConvolution", [1, grp, 0.0], [x, w, wb, b], [True, True, False, True], [gx, gw, wb, gb]),
    ]
    for op, scalars, ins, pd, g0 in runs:
        c = H.backward(CPU, op, scalars, [pad, stride, dil], ins, [dy], pd, [accum] * len(ins), g0)
        g = H.backward(B200, op, scalars, [pad, stride, dil], ins, [dy], pd, [accum] * len(ins), g0)
        for i, p in enumerate(pd):
            if p or (op == "BinaryConnectConvolution" and i == 2):
                assert cases.rel_rms(g[0][i], c[0][i]) < 1e-5, (op, i)
            else:
                assert np.array_equal(bits(g[0][i]), bits(c[0][i])), (op, i)


# ---- sibling quantization functions through nnabla's registry ---------------

@pytest.mark.parametrize("op", ["BinarySigmoid", "BinaryTanh"])
@pytest.mark.parametrize("accum", [False, True])
def test_binary_activations(op, accum):
    x = cases.binary_act_input()
    dy, dx0 = cases.grad_inputs(x)
    c, g = both(op, [], [], [x])
    assert np.array_equal(bits(g[0][0]), bits(c[0][0]))
    c, g = both_backward(op, [], [x], dy, [True], [accum], [dx0])
    assert np.array_equal(bits(g[0][0]), bits(c[0][0]))


@pytest.mark.parametrize("shapes,round_mode,narrow,dtype", cases.QL_GRID[::3])
def test_quantize_linear(shapes, round_mode, narrow, dtype):
    x, scale, zp = cases.quantize_linear_inputs(*shapes)
    c, g = both("QuantizeLinear", [round_mode == "HALF_TO_EVEN", narrow, dtype], [], [x, scale, zp])
    assert np.array_equal(bits(g[0][0]), bits(c[0][0]))
    assert np.array_equal(bits(g[1][2]), bits(c[1][2]))  # zero point rounded and saturated in place


@pytest.mark.parametrize("shapes", cases.QL_SHAPES)
@pytest.mark.parametrize("accum", [False, True])
def test_linear_backward_and_dequantize(shapes, accum):
    x, scale, zp = cases.quantize_linear_inputs(*shapes)
    dy, dx0 = cases.grad_inputs(x)
    c, g = both("DequantizeLinear", [], [], [x, scale, zp])
    assert np.array_equal(bits(g[0][0]), bits(c[0][0]))
    g0 = [dx0, np.zeros_like(scale), np.zeros_like(zp)]
    for op, scalars in (("QuantizeLinear", [0, 0, 1]), ("DequantizeLinear", [])):
        c, g = both_backward(op, scalars, [x, scale, zp], dy, [True, False, False], [accum, False, False], g0)
        assert np.array_equal(bits(g[0][0]), bits(c[0][0])), op


@pytest.mark.parametrize("rate", [0.0, 0.5, 0.9, 1.0])
def test_prune(rate):
    rng = np.random.RandomState(5)
    x = rng.randn(3, 7, 11).astype(np.float32)
    x.reshape(-1)[::9] = 0.0
    dy, dx0 = cases.grad_inputs(x)
    c, g = both("Prune", [rate], [], [x])
    assert np.array_equal(bits(g[0][0]), bits(c[0][0]))
    for accum in (False, True):
        c, g = both_backward("Prune", [rate], [x], dy, [True], [accum], [dx0])
        assert np.array_equal(bits(g[0][0]), bits(c[0][0]))
