"""Pins the C restatement (oracle/oracle_*.c) against the reference's own
compiled CPU functions (oracle/_ref/libnnabla_ref.so, built from the reference
checkout by `make -C oracle ref`). Bit-exact for the quantizers and signs; to
rounding for reductions and contractions (the reference sums with Eigen)."""
import numpy as np
import pytest

import cases
from oracle import oracle, ref

pytestmark = pytest.mark.skipif(not ref.available(), reason="reference CPU library not built")


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


@pytest.mark.parametrize("sign,n,delta", cases.FXP_GRID)
def test_fixed_point_quantize(sign, n, delta):
    n_eff = n - 1 if sign else n
    x = np.concatenate([cases.fxp_input().ravel(), cases.edge_values_fxp(np.float32(delta), n_eff)])
    want = ref.fixed_point_quantize(x, sign, n, delta)
    got = oracle.fixed_point_quantize(x, sign, n, delta)
    assert np.array_equal(bits(got), bits(want))


def test_fixed_point_quantize_configs():
    rng = np.random.RandomState(0)
    x = rng.uniform(-4, 4, 1 << 20).astype(np.float32)
    for delta in (2.0 ** -4, 2.0 ** -5, 2.0 ** -10):
        assert np.array_equal(bits(oracle.fixed_point_quantize(x, True, 8, delta)),
                              bits(ref.fixed_point_quantize(x, True, 8, delta)))


@pytest.mark.parametrize("sign,with_zero,n,m", cases.POW2_GRID + [(True, True, 8, 1), (False, False, 8, 1)])
def test_pow2_quantize(sign, with_zero, n, m):
    x = np.concatenate([cases.fxp_input().ravel(), cases.edge_values_pow2()])
    want = ref.pow2_quantize(x, sign, with_zero, n, m)
    got = oracle.pow2_quantize(x, sign, with_zero, n, m)
    assert np.array_equal(bits(got), bits(want))


def test_pow2_threshold_table_is_monotone():
    t, bad = oracle.pow2_thresholds()
    assert bad == 0
    assert t.shape == (254,)
    # the cut sits near sqrt(2): mantissa field 0x3504f3
    assert np.all(np.abs(t.astype(np.int64) - 0x3504f3) < 64)


@pytest.mark.parametrize("shapes,decay,x_min_max,ema", cases.MINMAX_GRID)
def test_min_max_quantize(shapes, decay, x_min_max, ema):
    x, qr_min, qr_max, ql_min, ql_max = cases.minmax_inputs(*shapes)
    wy, wmin, wmax = ref.min_max_quantize(x, qr_min, qr_max, ql_min, ql_max, decay, x_min_max, ema, True, 0.01)
    gy, gmin, gmax, _ = oracle.min_max_quantize(x, qr_min, qr_max, ql_min, ql_max, decay, x_min_max, ema, 0.01)
    assert np.array_equal(bits(gmin), bits(wmin))
    assert np.array_equal(bits(gmax), bits(wmax))
    assert np.array_equal(bits(gy), bits(wy))


@pytest.mark.parametrize("case", cases.minmax_zero_sign_cases(), ids=lambda c: c[0])
@pytest.mark.parametrize("ema", [False, True])
def test_min_max_quantize_zero_extrema(case, ema):
    """Signed zeros as the minimum / maximum (first one in scan order wins) and the +-1e8 start values."""
    _, x, qs = case
    q = lambda v: np.full(qs, v, np.float32)
    wy, wmin, wmax = ref.min_max_quantize(x, q(-0.5), q(0.5), q(0), q(255), 0.9, True, ema, True, 0.01)
    gy, gmin, gmax, _ = oracle.min_max_quantize(x, q(-0.5), q(0.5), q(0), q(255), 0.9, True, ema, 0.01)
    assert np.array_equal(bits(gmin), bits(wmin))
    assert np.array_equal(bits(gmax), bits(wmax))
    assert np.array_equal(bits(gy), bits(wy))


def test_min_max_quantize_config_and_eps_nudge():
    rng = np.random.RandomState(0)
    x = rng.uniform(-4, 4, (1 << 18,)).astype(np.float32)
    one = lambda v: np.array([v], np.float32)
    wy, _, wmax = ref.min_max_quantize(x, one(-4), one(4), one(0), one(255))
    gy, _, gmax, sc = oracle.min_max_quantize(x, one(-4), one(4), one(0), one(255))
    assert np.array_equal(bits(gy), bits(wy)) and np.array_equal(bits(gmax), bits(wmax))
    assert sc[0] == np.float32(0.03137255)
    # range narrower than eps: qr_max is pushed to qr_min + eps and written back
    wy, _, wmax = ref.min_max_quantize(x, one(0.5), one(0.501), one(0), one(255))
    gy, _, gmax, _ = oracle.min_max_quantize(x, one(0.5), one(0.501), one(0), one(255))
    assert np.array_equal(bits(gy), bits(wy)) and np.array_equal(bits(gmax), bits(wmax))
    assert gmax[0] == np.float32(0.5) + np.float32(0.01)


@pytest.mark.parametrize("alpha", cases.QZT)
def test_sign(alpha):
    x = np.concatenate([cases.fxp_input().ravel(), np.array([0.0, -0.0, np.nan, np.inf, -np.inf, 1e-45, -1e-45], np.float32)])
    assert np.array_equal(bits(oracle.sign(x, alpha)), bits(ref.sign(x, alpha)))


@pytest.mark.parametrize("xs,ws,base_axis", cases.AFFINE_CASES)
@pytest.mark.parametrize("qzt", cases.QZT)
@pytest.mark.parametrize("bias", [True, False])
def test_binary_weight_and_connect_affine(xs, ws, base_axis, qzt, bias):
    x, w, b = cases.affine_inputs(xs, ws, with_zeros=True)
    b = b if bias else None
    wy, wwb, wal = ref.binary_weight_affine(x, w, b, base_axis, qzt)
    gy, gwb, gal = oracle.binary_weight_affine(x, w, b, base_axis, qzt)
    assert np.array_equal(bits(gwb), bits(wwb))
    np.testing.assert_allclose(gal, wal, rtol=1e-6)
    assert gy.shape == wy.shape and cases.rel_rms(gy, wy) < 1e-6
    wy, wwb = ref.binary_connect_affine(x, w, b, base_axis, qzt)
    gy, gwb = oracle.binary_connect_affine(x, w, b, base_axis, qzt)
    assert np.array_equal(bits(gwb), bits(wwb))
    assert gy.shape == wy.shape and cases.rel_rms(gy, wy) < 1e-6


@pytest.mark.parametrize("xs,ws,pad,stride,dilation,group", cases.CONV_CASES)
@pytest.mark.parametrize("qzt", [1.0, 0.0])
def test_binary_weight_and_connect_convolution(xs, ws, pad, stride, dilation, group, qzt):
    x, w, b = cases.conv_inputs(xs, ws, with_zeros=True)
    wy, wwb, wal = ref.binary_weight_convolution(x, w, b, 1, pad, stride, dilation, group, qzt)
    gy, gwb, gal = oracle.binary_weight_convolution(x, w, b, pad, stride, dilation, group, qzt)
    assert np.array_equal(bits(gwb), bits(wwb))
    np.testing.assert_allclose(gal, wal, rtol=1e-6)
    assert gy.shape == wy.shape and cases.rel_rms(gy, wy) < 1e-6
    wy, wwb = ref.binary_connect_convolution(x, w, None, 1, pad, stride, dilation, group, qzt)
    gy, gwb = oracle.binary_connect_convolution(x, w, None, pad, stride, dilation, group, qzt)
    assert np.array_equal(bits(gwb), bits(wwb))
    assert cases.rel_rms(gy, wy) < 1e-6


def test_companions():
    rng = np.random.RandomState(cases.SEED)
    x = rng.randn(2, 6, 9, 11).astype(np.float32)
    beta, gamma, mean = (rng.randn(1, 6, 1, 1).astype(np.float32) for _ in range(3))
    var = (rng.rand(1, 6, 1, 1) + 0.1).astype(np.float32)
    assert np.array_equal(bits(oracle.batch_norm_inference(x, beta, gamma, mean, var, 1e-5)),
                          bits(ref.batch_normalization(x, beta, gamma, mean, var, eps=1e-5)))
    assert np.array_equal(bits(oracle.relu(x)), bits(ref.relu(x)))
    assert np.array_equal(bits(oracle.add2(x, x[::-1].copy())), bits(ref.add2(x, x[::-1].copy())))
    for k, s, p, ib in [((3, 3), (2, 2), (1, 1), True), ((2, 2), (2, 2), (0, 0), True), ((3, 3), (2, 2), (0, 0), False)]:
        assert np.array_equal(bits(oracle.max_pooling(x, k, s, ib, p)), bits(ref.max_pooling(x, k, s, ib, p)))
    assert np.array_equal(bits(oracle.global_average_pooling(x)), bits(ref.global_average_pooling(x)))
    w = rng.randn(6, 6, 3, 3).astype(np.float32)
    assert cases.rel_rms(oracle.convolution(x, w, None, (1, 1)), ref.convolution(x, w, None, 1, (1, 1))) < 1e-6
    xa, wa, ba = cases.affine_inputs((3, 5, 7), (35, 40))
    assert cases.rel_rms(oracle.affine(xa, wa, ba), ref.affine(xa, wa, ba)) < 1e-6
