"""GPU parity of the quantizers' backward passes, through the C ABI: input
gradients bit-exact against the golden vectors made by the reference's own
Function::backward and against the oracle on sizes that exercise the
vector body, tails and misaligned buffers; the two range gradients of
MinMaxQuantize (fp32 sums) to rounding."""
import numpy as np
import pytest
import torch

import backward_cases
import cases
from golden_util import bits
from oracle import oracle

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).cuda()


def host(t):
    return t.cpu().numpy()


@pytest.fixture(scope="module")
def F():
    from nnabla_b200 import _capi, functions
    _capi.call("nb200_check_device")
    return functions


class Device:
    """The CUDA path behind the oracle's numpy signatures."""

    def __init__(self, F):
        self.F = F

    def fixed_point_quantize_backward(self, x, dy, sign, n, delta, fine, accum, dx0):
        return host(self.F.fixed_point_quantize_backward(dev(x), dev(dy), sign, n, delta, fine, accum, dev(dx0)))

    def pow2_quantize_backward(self, x, dy, sign, wz, n, m, fine, accum, dx0):
        return host(self.F.pow2_quantize_backward(dev(x), dev(dy), sign, wz, n, m, fine, accum, dev(dx0)))

    def min_max_quantize(self, x, qmin, qmax, lmin, lmax, decay, xmm, ema, eps):
        a, b = dev(qmin), dev(qmax)
        y = self.F.min_max_quantize(dev(x), a, b, dev(lmin), dev(lmax), decay, xmm, ema, True, eps)
        return host(y), host(a), host(b)

    def min_max_quantize_backward(self, x, qmin, qmax, lmin, lmax, dy, xmm, ema, fine, pd, ac, g0):
        r = self.F.min_max_quantize_backward(dev(x), dev(qmin), dev(qmax), dev(lmin), dev(lmax), dev(dy), xmm, ema,
                                             fine, pd, ac, [dev(g) for g in g0])
        return tuple(host(t) for t in r)


@pytest.mark.parametrize("i", range(len(cases.FXP_GRID)))
@pytest.mark.parametrize("fine,accum", backward_cases.FLAGS)
def test_fxp_backward_golden(F, i, fine, accum):
    backward_cases.check_fxp(Device(F), i, fine, accum)


@pytest.mark.parametrize("i", range(len(backward_cases.POW2_CASES)))
@pytest.mark.parametrize("fine,accum", backward_cases.FLAGS)
def test_pow2_backward_golden(F, i, fine, accum):
    backward_cases.check_pow2(Device(F), i, fine, accum)


@pytest.mark.parametrize("i", range(len(cases.MINMAX_GRID)))
@pytest.mark.parametrize("fine,accum", backward_cases.FLAGS)
def test_minmax_backward_golden(F, i, fine, accum):
    backward_cases.check_minmax(Device(F), i, fine, accum)


@pytest.mark.parametrize("size", cases.VEC_TAIL_SIZES + [1 << 20])
@pytest.mark.parametrize("offset", [0, 1])
@pytest.mark.parametrize("accum", [False, True])
def test_backward_tails_and_misalignment(F, size, offset, accum):
    rng = np.random.RandomState(size + offset)
    x = (rng.randn(size + offset) * 6).astype(np.float32)
    dy = rng.randn(size + offset).astype(np.float32)
    dx0 = rng.randn(size + offset).astype(np.float32)
    xd, dyd = dev(x)[offset:], dev(dy)[offset:]
    sl = slice(offset, None)
    got = F.fixed_point_quantize_backward(xd, dyd, True, 8, 2.0 ** -4, True, accum, dev(dx0)[offset:].contiguous())
    want = oracle.fixed_point_quantize_backward(x[sl], dy[sl], True, 8, 2.0 ** -4, True, accum, dx0[sl])
    assert np.array_equal(bits(host(got)), bits(want))
    got = F.pow2_quantize_backward(xd, dyd, True, True, 8, 1, True, accum, dev(dx0)[offset:].contiguous())
    want = oracle.pow2_quantize_backward(x[sl], dy[sl], True, True, 8, 1, True, accum, dx0[sl])
    assert np.array_equal(bits(host(got)), bits(want))
    got = F.pow2_quantize_backward(xd, dyd, False, False, 4, 0, False, accum, dev(dx0)[offset:].contiguous())
    want = oracle.pow2_quantize_backward(x[sl], dy[sl], False, False, 4, 0, False, accum, dx0[sl])
    assert np.array_equal(bits(host(got)), bits(want))


def test_pow2_backward_extreme_ranges(F):
    """p_max beyond every float (no gradient is blocked) and below every float
    (every non-zero input is blocked)."""
    x = np.concatenate([cases.edge_values_pow2(), np.array([np.nan, 0.0, -0.0], np.float32)])
    dy, dx0 = cases.grad_inputs(x)
    for m in (200, 128, 127, -140, -149, -150, -300):
        want = oracle.pow2_quantize_backward(x, dy, True, True, 4, m, True, False, dx0)
        got = F.pow2_quantize_backward(dev(x), dev(dy), True, True, 4, m, True, False)
        assert np.array_equal(bits(host(got)), bits(want)), m


def test_minmax_backward_large_per_tensor(F):
    """BASELINE configs[1] ranges on 2^22 elements: dx bit-exact, range gradients against a float64 sum."""
    rng = np.random.RandomState(0)
    n = 1 << 22
    x = rng.uniform(-4.5, 4.5, n).astype(np.float32)
    dy = rng.randn(n).astype(np.float32)
    one = lambda v: np.array([v], np.float32)
    qmin, qmax, lmin, lmax = one(-4), one(4), one(0), one(255)
    _, fmin, fmax, _ = oracle.min_max_quantize(x, qmin, qmax, lmin, lmax)
    want_dx, _, _ = oracle.min_max_quantize_backward(x, fmin, fmax, lmin, lmax, dy)
    dx, gmin, gmax = F.min_max_quantize_backward(dev(x), dev(fmin), dev(fmax), dev(lmin), dev(lmax), dev(dy))
    assert np.array_equal(bits(host(dx)), bits(want_dx))
    # nudged range (min_max_quantize.cpp:362-390) in fp32: scale 8/255, zero point round(0 - (-4 / scale)) = 127
    scale = np.float32(8) / np.float32(255)
    zp = np.round(np.float32(0) - np.float32(-4) / scale)
    m, M = (np.float32(0) - zp) * scale, (np.float32(255) - zp) * scale
    lo64 = dy[x < m].astype(np.float64).sum()
    hi64 = dy[x > M].astype(np.float64).sum()
    assert abs(float(host(gmin)[0]) - lo64) < 1e-3 and abs(float(host(gmax)[0]) - hi64) < 1e-3


def test_backward_argument_errors(F):
    x = torch.zeros(8, device="cuda")
    with pytest.raises(RuntimeError):
        F.fixed_point_quantize_backward(x, torch.zeros(9, device="cuda"))
    with pytest.raises(RuntimeError):
        F.fixed_point_quantize_backward(x, x, accum=True)
    with pytest.raises(RuntimeError):
        F.fixed_point_quantize_backward(x, x, n=0)
    with pytest.raises(RuntimeError):
        F.pow2_quantize_backward(x, x, n=1)
