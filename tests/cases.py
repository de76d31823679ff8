"""Seeded inputs shared by the oracle, golden-fixture and GPU parity tests.

The parameter grids restate the reference's own test files
(python/test/function/test_fixed_point_quantize.py:65-92,
test_pow2_quantize.py:73-101, test_min_max_quantize.py:112-128,
test_binary_weight_affine.py:67-93, test_binary_weight_convolution.py:72-98),
seed 313, plus the edge values those tests do not reach.
"""
import itertools

import numpy as np

SEED = 313


def f32(bits):
    return np.array(bits, dtype=np.uint32).view(np.float32)


def edge_values_fxp(delta, n_eff):
    """Half-way points k*delta + delta/2 and their neighbours, the limits,
    signed zeros, denormals, infinities (no NaN: int(NaN) is undefined in
    fixed_point_quantize.cpp:61)."""
    k = np.arange(0, 2 ** n_eff + 2, dtype=np.float64)
    half = ((k + 0.5) * delta).astype(np.float32)
    vals = [half, np.nextafter(half, np.float32(np.inf)), np.nextafter(half, np.float32(-np.inf)),
            (k * delta).astype(np.float32)]
    mx = np.float32((2 ** n_eff - 1) * delta)
    extra = np.array([0.0, -0.0, mx, -mx, np.nextafter(mx, np.float32(np.inf)), np.nextafter(mx, np.float32(0)),
                      np.inf, -np.inf, 1e-45, -1e-45, 1e-38, -1e-38, 3.4e38, -3.4e38,
                      0.49999997 * delta, 0.5 * delta, -0.03, 0.09375, 9, -9], dtype=np.float32)
    v = np.concatenate(vals + [extra])
    return np.concatenate([v, -v]).astype(np.float32)


def edge_values_pow2():
    """Values around sqrt(2)*2^e for every normal exponent, powers of two,
    denormals, zeros, infinities."""
    out = []
    for e in range(-126, 128):
        c = np.float32(np.sqrt(2.0)) * np.float32(2.0) ** np.float32(e) if e < 127 else np.float32(2.0) ** 127 * np.float32(1.4142135)
        cb = np.array([c], np.float32).view(np.uint32)[0]
        if not np.isfinite(c):
            continue
        out.append(f32(np.arange(int(cb) - 40, int(cb) + 41, dtype=np.int64).astype(np.uint32)))
        out.append(np.array([np.float32(2.0) ** np.float32(e)], np.float32))
    extra = np.array([0.0, -0.0, np.inf, -np.inf, 1e-45, -1e-45, 5e-39, 1.1754942e-38, 1.41421, 9, -0.001,
                      3.4e38, 2.0, 1.9999999, 2.0000002], dtype=np.float32)
    v = np.concatenate(out + [extra]).astype(np.float32)
    return np.concatenate([v, -v])


def pow2_backward_edges(m):
    """Inputs around the only place where Pow2Quantize's gradient factor changes
    (the snap from 2^m to 2^(m+1)), plus NaNs, whose factor stays 1."""
    c = np.array([np.sqrt(2.0) * 2.0 ** m], np.float32).view(np.uint32)[0]
    near = f32(np.arange(int(c) - 300, int(c) + 301, dtype=np.int64).astype(np.uint32))
    v = np.concatenate([near, np.array([np.nan, 2.0 ** m, 2.0 ** (m + 1), 2.0 ** (m + 1) * 0.99999], np.float32)])
    return np.concatenate([v, -v]).astype(np.float32)


def grad_inputs(x, seed=7):
    """Output gradient (with zeros and sign flips) and an initial input gradient for backward cases."""
    rng = np.random.RandomState(seed)
    dy = rng.randn(*x.shape).astype(np.float32)
    dy.reshape(-1)[::13] = 0.0
    dy.reshape(-1)[5::17] *= -1.0
    dx0 = rng.randn(*x.shape).astype(np.float32)
    return dy, dx0


def fxp_backward_input(delta, n_eff):
    x = np.concatenate([fxp_input((2, 3, 50)).ravel(), edge_values_fxp(np.float32(delta), n_eff)])
    return x[~np.isnan(x)]


def pow2_backward_input(m):
    return np.concatenate([fxp_input((2, 3, 50)).ravel(), edge_values_pow2(), pow2_backward_edges(m)])


FXP_GRID = list(itertools.product([False, True], [3, 8], [2.0 ** -7, 0.005]))   # sign, n, delta
POW2_GRID = list(itertools.product([False, True], [False, True], [3, 5], [0, 1]))  # sign, with_zero, n, m
MINMAX_SHAPES = [((4, 8, 16, 16), (1, 1, 1, 1)), ((4, 8, 16, 16), (1, 8, 1, 1)), ((16, 8, 3, 3), (16, 1, 1, 1))]
MINMAX_GRID = list(itertools.product(MINMAX_SHAPES, [0.999, 0.9], [True, False], [True, False]))  # decay,x_min_max,ema
VEC_TAIL_SIZES = [0, 1, 3, 4, 5, 31, 1023, 1025, 4099]


def fxp_input(shape=(2, 3, 4, 33)):
    rng = np.random.RandomState(SEED)
    return (rng.randn(*shape) * 2).astype(np.float32)


def minmax_zero_sign_cases():
    """Inputs whose min or max is a zero, or lies outside the +-1e8 start values of the
    reference's Min / Max scans (src/nbla/function/generic/max.cpp:49-57): (name, x, q_shape).
    The sign of a zero extremum is that of the FIRST zero in scan order, and it is written
    back into qr_min / qr_max. Sizes span one block and several blocks of the device reduction."""
    f32 = np.float32
    rng = np.random.RandomState(SEED + 1)
    out = []
    for n in (64, 70000):
        neg = -np.abs(rng.randn(n)).astype(f32) - f32(0.25)
        pos = np.abs(rng.randn(n)).astype(f32) + f32(0.25)
        a = neg.copy(); a[n // 3] = f32(-0.0)                     # max is -0.0 alone
        b = neg.copy(); b[n // 3] = f32(-0.0); b[n // 3 + 7] = f32(0.0)   # -0.0 first, then +0.0
        c = neg.copy(); c[n // 3] = f32(0.0); c[n - 2] = f32(-0.0)        # +0.0 first
        d = pos.copy(); d[n // 2] = f32(-0.0)                     # min is -0.0 alone
        e = pos.copy(); e[5] = f32(0.0); e[n - 1] = f32(-0.0)     # min: +0.0 first
        g = pos.copy(); g[n - 1] = f32(0.0); g[3] = f32(-0.0)     # min: -0.0 first
        h = np.concatenate([pos[: n // 2], neg[: n // 2]]); h[1] = f32(-0.0)  # zero inside the range
        for name, x in (("max-0", a), ("max-0+0", b), ("max+0-0", c), ("min-0", d), ("min+0-0", e), ("min-0+0", g),
                        ("mixed", h)):
            out.append(("%s/%d" % (name, n), x.reshape(1, -1), (1, 1)))
    # per-channel ranges: channel 0 all non-positive with -0.0, channel 1 all non-negative with -0.0 late
    x = rng.randn(3, 4, 50).astype(f32)
    x[:, 0] = -np.abs(x[:, 0]) - f32(0.5); x[2, 0, 7] = f32(-0.0)
    x[:, 1] = np.abs(x[:, 1]) + f32(0.5); x[0, 1, 9] = f32(0.0); x[1, 1, 0] = f32(-0.0)
    out.append(("per-channel", x, (1, 4, 1)))
    # beyond the scan's start values: all below -1e8 (max stays -1e8), all above +1e8 (min stays +1e8)
    out.append(("below-1e8", np.array([[-3e8, -2e8, -5e8]], f32), (1, 1)))
    out.append(("above+1e8", np.array([[3e8, 2e8, 5e8]], f32), (1, 1)))
    return out


def minmax_inputs(x_shape, q_shape):
    rng = np.random.RandomState(SEED)
    x = rng.randn(*x_shape).astype(np.float32)
    qr_min = (-0.5 * rng.rand(*q_shape)).astype(np.float32)
    qr_max = (+0.5 * rng.rand(*q_shape)).astype(np.float32)
    ql_min = np.zeros(q_shape, np.float32)
    ql_max = np.full(q_shape, 255, np.float32)
    return x, qr_min, qr_max, ql_min, ql_max


# (x shape, w shape, base_axis) as in test_binary_weight_affine.py, plus a wider case
AFFINE_CASES = [((2, 4, 3), (12, 2, 3), 1), ((2, 4), (4, 4), 1), ((3, 5, 7), (35, 40), 1), ((2, 3, 8), (8, 16), 2)]
QZT = [0.0, -1.0, 1.0]

# (x shape, w shape, pad, stride, dilation, group)
CONV_CASES = [
    ((2, 2, 10, 10), (4, 2, 3, 2), (0, 0), (1, 2), (2, 1), 1),
    ((2, 4, 10, 10), (4, 2, 3, 2), (0, 1), (1, 2), (2, 1), 2),
    ((3, 8, 9, 9), (16, 8, 3, 3), (1, 1), (1, 1), (1, 1), 1),
    ((2, 8, 12, 12), (8, 8, 1, 1), (0, 0), (2, 2), (1, 1), 1),
    ((1, 16, 7, 7), (32, 16, 3, 3), (1, 1), (2, 2), (1, 1), 1),
]


def affine_inputs(xs, ws, with_zeros=False):
    rng = np.random.RandomState(SEED)
    x = rng.randn(*xs).astype(np.float32)
    w = rng.randn(*ws).astype(np.float32)
    b = rng.randn(*ws[1:]).astype(np.float32)
    if with_zeros:
        w.reshape(-1)[::7] = 0.0
        w.reshape(-1)[3::11] = -0.0
    return x, w, b


def conv_inputs(xs, ws, with_zeros=False):
    rng = np.random.RandomState(SEED)
    x = rng.randn(*xs).astype(np.float32)
    w = rng.randn(*ws).astype(np.float32)
    b = rng.randn(ws[0]).astype(np.float32)
    if with_zeros:
        w.reshape(-1)[::5] = 0.0
    return x, w, b


def rel_rms(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.sqrt(np.mean((a - b) ** 2)) / max(np.sqrt(np.mean(b ** 2)), 1e-30))


# ---- sibling quantization functions ---------------------------------------------
def binary_act_input():
    rng = np.random.RandomState(SEED)
    x = (rng.randn(2, 3, 4, 37) * 1.5).astype(np.float32)
    edges = np.array([0.0, -0.0, 1.0, -1.0, 0.99999994, -0.99999994, 1.0000001, np.inf, -np.inf, np.nan, 1e-45, -1e-45],
                     np.float32)
    return np.concatenate([x.ravel(), edges])


# (x shape, scale shape, zero-point shape)
QL_SHAPES = [((4, 6, 5, 5), (1, 1, 1, 1), (1, 1, 1, 1)), ((4, 6, 5, 5), (1, 6, 1, 1), (1, 1, 1, 1)),
             ((4, 6, 5, 5), (1, 6, 1, 1), (1, 6, 1, 1)), ((8, 33), (8, 1), (1, 1))]
QL_GRID = list(itertools.product(QL_SHAPES, ["HALF_AWAY_FROM_ZERO", "HALF_TO_EVEN"], [False, True], [1, 2]))


def quantize_linear_inputs(xs, ss, zs):
    rng = np.random.RandomState(SEED)
    x = (rng.randn(*xs) * 40).astype(np.float32)
    x.reshape(-1)[::7] = np.round(x.reshape(-1)[::7]) + 0.5      # exact halves after division by a power of two
    scale = (2.0 ** rng.randint(-2, 2, size=ss)).astype(np.float32)
    scale.reshape(-1)[::2] *= np.float32(1.3)
    zp = (rng.randn(*zs) * 100 + 0.5 * rng.randint(0, 2, size=zs)).astype(np.float32)
    return x, scale, zp
