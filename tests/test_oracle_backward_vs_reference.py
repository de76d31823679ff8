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
