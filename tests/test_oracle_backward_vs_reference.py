"""Pins the C restatement of the quantizers' backward passes
(oracle/oracle_backward.c) against Function::backward of the reference's own
compiled CPU functions (oracle/_ref/libnnabla_ref.so). Bit-exact for the input
gradients; to rounding for the two range gradients of MinMaxQuantize (fp32
sums whose order the reference takes from Eigen)."""
import numpy as np
import pytest

import cases
from oracle import oracle, ref

pytestmark = pytest.mark.skipif(not ref.available(), reason="reference CPU library not built")


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


grads_for = cases.grad_inputs


@pytest.mark.parametrize("sign,n,delta", cases.FXP_GRID)
@pytest.mark.parametrize("fine", [True, False])
@pytest.mark.parametrize("accum", [False, True])
def test_fixed_point_quantize_backward(sign, n, delta, fine, accum):
    n_eff = n - 1 if sign else n
    x = np.concatenate([cases.fxp_input().ravel(), cases.edge_values_fxp(np.float32(delta), n_eff)])
    x = x[~np.isnan(x)]
    dy, dx0 = grads_for(x)
    want = ref.fixed_point_quantize_backward(x, dy, sign, n, delta, fine, accum, dx0)
    got = oracle.fixed_point_quantize_backward(x, dy, sign, n, delta, fine, accum, dx0)
    assert np.array_equal(bits(got), bits(want))


@pytest.mark.parametrize("sign,with_zero,n,m", cases.POW2_GRID + [(True, True, 8, 1), (False, False, 8, 1)])
@pytest.mark.parametrize("fine", [True, False])
@pytest.mark.parametrize("accum", [False, True])
def test_pow2_quantize_backward(sign, with_zero, n, m, fine, accum):
    x = np.concatenate([cases.fxp_input().ravel(), cases.edge_values_pow2(), cases.pow2_backward_edges(m)])
    dy, dx0 = grads_for(x)
    want = ref.pow2_quantize_backward(x, dy, sign, with_zero, n, m, fine, accum, dx0)
    got = oracle.pow2_quantize_backward(x, dy, sign, with_zero, n, m, fine, accum, dx0)
    assert np.array_equal(bits(got), bits(want))


@pytest.mark.parametrize("shapes,decay,x_min_max,ema", cases.MINMAX_GRID)
@pytest.mark.parametrize("fine", [True, False])
@pytest.mark.parametrize("accum", [False, True])
def test_min_max_quantize_backward(shapes, decay, x_min_max, ema, fine, accum):
    x, qr_min, qr_max, ql_min, ql_max = cases.minmax_inputs(*shapes)
    dy, dx0 = grads_for(x)
    rng = np.random.RandomState(3)
    g0 = [dx0, rng.randn(*qr_min.shape).astype(np.float32), rng.randn(*qr_min.shape).astype(np.float32)]
    ranges = not (x_min_max or ema)
    pd = (True, ranges, ranges)
    ac = (accum, accum, accum)
    wdx, wgmin, wgmax = ref.min_max_quantize_backward(x, qr_min, qr_max, ql_min, ql_max, dy, decay, x_min_max, ema,
                                                      fine, 0.01, pd, ac, g0)
    # the oracle's backward starts from the ranges the forward left behind
    _, fmin, fmax, _ = oracle.min_max_quantize(x, qr_min, qr_max, ql_min, ql_max, decay, x_min_max, ema, 0.01)
    gdx, ggmin, ggmax = oracle.min_max_quantize_backward(x, fmin, fmax, ql_min, ql_max, dy, x_min_max, ema, fine,
                                                         pd, ac, g0)
    assert np.array_equal(bits(gdx), bits(wdx))
    if ranges:
        per_q = x.size // qr_min.size
        tol = 1e-6 * per_q ** 0.5 * (np.abs(dy).max() + 1)
        assert np.allclose(ggmin, wgmin, rtol=1e-5, atol=tol)
        assert np.allclose(ggmax, wgmax, rtol=1e-5, atol=tol)
    else:
        assert np.array_equal(bits(ggmin), bits(g0[1])) and np.array_equal(bits(ggmax), bits(g0[2]))


def affine_grad_case(xs, ws, base_axis):
    x, w, b = cases.affine_inputs(xs, ws, with_zeros=True)
    rng = np.random.RandomState(1)
    dy = rng.randn(*(tuple(xs[:base_axis]) + tuple(ws[1:]))).astype(np.float32)
    g0 = [rng.randn(*xs).astype(np.float32), rng.randn(*ws).astype(np.float32),
          rng.randn(*ws[1:]).astype(np.float32)]
    return x, w, b, dy, g0


@pytest.mark.parametrize("xs,ws,base_axis", cases.AFFINE_CASES)
@pytest.mark.parametrize("accum", [False, True])
def test_affine_backward_family(xs, ws, base_axis, accum):
    x, w, b, dy, g0 = affine_grad_case(xs, ws, base_axis)
    ac = (accum,) * 3
    pairs = [
        (ref.affine_backward(x, w, b, dy, base_axis, accum=ac, grads=g0),
         oracle.affine_backward(x, w, dy, base_axis, accum=ac, grads=g0)),
        (ref.binary_weight_affine_backward(x, w, b, dy, base_axis, 1.0, accum=ac, grads=g0),
         oracle.binary_weight_affine_backward(x, w, dy, base_axis, 1.0, accum=ac, grads=g0)),
        (ref.binary_connect_affine_backward(x, w, b, dy, base_axis, 0.0, accum=ac, grads=g0),
         oracle.binary_connect_affine_backward(x, w, dy, base_axis, 0.0, accum=ac, grads=g0)),
    ]
    for want, got in pairs:
        for a, c in zip(got, want):
            assert cases.rel_rms(a, c) < 1e-6


def test_binary_weight_affine_backward_without_bias_and_partial_propagation():
    xs, ws, base_axis = cases.AFFINE_CASES[2]
    x, w, _, dy, g0 = affine_grad_case(xs, ws, base_axis)
    want = ref.binary_weight_affine_backward(x, w, None, dy, base_axis, 1.0, propagate_down=(True, False, False),
                                             grads=g0)
    got = oracle.binary_weight_affine_backward(x, w, dy, base_axis, 1.0, propagate_down=(True, False, False),
                                               grads=g0)
    assert cases.rel_rms(got[0], want[0]) < 1e-6
    assert np.array_equal(got[1], g0[1]) and np.array_equal(want[1], g0[1])  # weight gradient untouched


@pytest.mark.parametrize("xs,ws,pad,stride,dil,grp", cases.CONV_CASES)
@pytest.mark.parametrize("accum", [False, True])
def test_convolution_backward_family(xs, ws, pad, stride, dil, grp, accum):
    x, w, b = cases.conv_inputs(xs, ws, with_zeros=True)
    rng = np.random.RandomState(2)
    dy = rng.randn(*oracle.conv_out_shape(xs, ws, pad, stride, dil)).astype(np.float32)
    g0 = [rng.randn(*xs).astype(np.float32), rng.randn(*ws).astype(np.float32), rng.randn(ws[0]).astype(np.float32)]
    ac = (accum,) * 3
    pairs = [
        (ref.convolution_backward(x, w, b, dy, 1, pad, stride, dil, grp, accum=ac, grads=g0),
         oracle.convolution_backward(x, w, dy, pad, stride, dil, grp, accum=ac, grads=g0)),
        (ref.binary_weight_convolution_backward(x, w, b, dy, 1, pad, stride, dil, grp, 1.0, accum=ac, grads=g0),
         oracle.binary_weight_convolution_backward(x, w, dy, pad, stride, dil, grp, 1.0, accum=ac, grads=g0)),
        (ref.binary_connect_convolution_backward(x, w, b, dy, 1, pad, stride, dil, grp, 0.0, accum=ac, grads=g0),
         oracle.binary_connect_convolution_backward(x, w, dy, pad, stride, dil, grp, 0.0, accum=ac, grads=g0)),
    ]
    for want, got in pairs:
        for a, c in zip(got, want):
            assert cases.rel_rms(a, c) < 1e-6
