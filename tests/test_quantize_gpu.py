"""GPU parity of the elementwise quantizers, through the C ABI, against the
oracle (bit-exact) and the golden vectors produced by the reference."""
import numpy as np
import pytest
import torch

import cases
from golden_util import bits, golden, sha
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


@pytest.mark.parametrize("i", range(len(cases.FXP_GRID)))
def test_fxp_golden(F, i):
    g = golden()
    sign, n, delta = g[f"fxp{i}/args"]
    y = F.fixed_point_quantize(dev(g[f"fxp{i}/x"]), bool(sign), int(n), float(delta))
    assert np.array_equal(bits(host(y)), bits(g[f"fxp{i}/out"]))


@pytest.mark.parametrize("size", cases.VEC_TAIL_SIZES)
@pytest.mark.parametrize("offset", [0, 1, 3])
def test_fxp_tails_and_misalignment(F, size, offset):
    rng = np.random.RandomState(size + offset)
    x = (rng.randn(size + offset) * 3).astype(np.float32)
    xd = dev(x)[offset:]
    want = oracle.fixed_point_quantize(x[offset:], True, 8, 2.0 ** -4)
    y = F.fixed_point_quantize(xd, True, 8, 2.0 ** -4)
    assert np.array_equal(bits(host(y)), bits(want))
    # output with a different 16-byte phase than the input
    buf = torch.empty(size + 4, device="cuda")
    yo = buf[(offset + 1) % 4:][:size]
    F.fixed_point_quantize(xd, True, 8, 0.005, outputs=[yo])
    assert np.array_equal(bits(host(yo)), bits(oracle.fixed_point_quantize(x[offset:], True, 8, 0.005)))


def test_fxp_codes(F):
    rng = np.random.RandomState(1)
    x = (rng.randn(100003) * 3).astype(np.float32)
    for sign, n, delta in [(True, 8, 2.0 ** -5), (True, 8, 2.0 ** -10), (False, 7, 0.005), (True, 3, 0.25)]:
        y, k = F.fixed_point_quantize_with_codes(dev(x), sign, n, delta)
        want = oracle.fixed_point_quantize(x, sign, n, delta)
        assert np.array_equal(bits(host(y)), bits(want))
        kk = k.cpu().numpy().astype(np.float32)
        assert np.array_equal(kk * np.float32(delta), want)


def test_fxp_inplace_and_cfg_digest(F):
    g = golden()
    rng = np.random.RandomState(0)
    x = rng.uniform(-4, 4, 1 << 20).astype(np.float32)
    xd = dev(x)
    F.fixed_point_quantize(xd, True, 8, 2.0 ** -4, outputs=[xd])
    assert np.array_equal(sha(host(xd)), g["cfg2_fxp/sha"])


@pytest.mark.parametrize("i", range(len(cases.POW2_GRID) + 1))
def test_pow2_golden(F, i):
    g = golden()
    sign, wz, n, m = g[f"pow2_{i}/args"]
    y = F.pow2_quantize(dev(g["pow2/x"]), bool(sign), bool(wz), int(n), int(m))
    assert np.array_equal(bits(host(y)), bits(g[f"pow2_{i}/out"]))


@pytest.mark.parametrize("sign,with_zero,n,m", [(True, False, 8, 1), (False, False, 8, 0), (True, True, 8, 1),
                                                (False, True, 9, 3), (True, False, 9, -2)])
def test_pow2_wide_ranges_vs_oracle(F, sign, with_zero, n, m):
    """p_min underflows to 0 for large n: the snapped value of tiny and
    denormal inputs is then visible in the output."""
    x = np.concatenate([cases.edge_values_pow2(), cases.fxp_input().ravel()])
    y = F.pow2_quantize(dev(x), sign, with_zero, n, m)
    assert np.array_equal(bits(host(y)), bits(oracle.pow2_quantize(x, sign, with_zero, n, m)))


def test_pow2_denormal_sweep_and_cfg_digest(F):
    g = golden()
    d = np.arange(1, 1 << 23, 997, dtype=np.uint32).view(np.float32)  # denormals
    y = F.pow2_quantize(dev(d), True, False, 9, 1)
    assert np.array_equal(bits(host(y)), bits(oracle.pow2_quantize(d, True, False, 9, 1)))
    rng = np.random.RandomState(0)
    x = rng.uniform(-4, 4, 1 << 20).astype(np.float32)
    assert np.array_equal(sha(host(F.pow2_quantize(dev(x), True, True, 8, 1))), g["cfg2_pow2/sha"])


@pytest.mark.parametrize("size", cases.VEC_TAIL_SIZES)
def test_pow2_tails(F, size):
    rng = np.random.RandomState(size)
    x = (rng.randn(size + 1) * 3).astype(np.float32)
    y = F.pow2_quantize(dev(x)[1:], True, True, 5, 1)
    assert np.array_equal(bits(host(y)), bits(oracle.pow2_quantize(x[1:], True, True, 5, 1)))


@pytest.mark.parametrize("i", range(len(cases.MINMAX_GRID)))
def test_minmax_golden(F, i):
    g = golden()
    decay, xmm, ema, eps = g[f"minmax{i}/args"]
    x, qmin, qmax, lmin, lmax = cases.minmax_inputs(tuple(g[f"minmax{i}/xshape"]), tuple(g[f"minmax{i}/qshape"]))
    dmin, dmax = dev(qmin), dev(qmax)
    y = F.min_max_quantize(dev(x), dmin, dmax, dev(lmin), dev(lmax), float(decay), bool(xmm), bool(ema), True,
                           float(eps))
    assert np.array_equal(bits(host(dmin)), bits(g[f"minmax{i}/out_qr_min"]))
    assert np.array_equal(bits(host(dmax)), bits(g[f"minmax{i}/out_qr_max"]))
    assert np.array_equal(sha(host(y)), g[f"minmax{i}/out_sha"])


@pytest.mark.parametrize("case", cases.minmax_zero_sign_cases(), ids=lambda c: c[0])
@pytest.mark.parametrize("ema", [False, True])
def test_minmax_zero_extrema(F, case, ema):
    """x_min_max with a signed zero as the extremum: the first zero in the reference's scan order
    gives qr_min / qr_max its sign (one block and several blocks of the device reduction), and the
    scans start from +-1e8 as the reference's Min / Max do."""
    _, x, qs = case
    q = lambda v: np.full(qs, v, np.float32)
    dmin, dmax = dev(q(-0.5)), dev(q(0.5))
    y = F.min_max_quantize(dev(x), dmin, dmax, dev(q(0)), dev(q(255)), 0.9, True, ema, True, 0.01)
    wy, wmin, wmax, _ = oracle.min_max_quantize(x, q(-0.5), q(0.5), q(0), q(255), 0.9, True, ema, 0.01)
    assert np.array_equal(bits(host(dmin)), bits(wmin))
    assert np.array_equal(bits(host(dmax)), bits(wmax))
    assert np.array_equal(bits(host(y)), bits(wy))


def test_minmax_cfg_digest_tails_and_errors(F):
    g = golden()
    rng = np.random.RandomState(0)
    x = rng.uniform(-4, 4, 1 << 20).astype(np.float32)
    one = lambda v: dev(np.array([v], np.float32))
    y = F.min_max_quantize(dev(x), one(-4), one(4), one(0), one(255))
    assert np.array_equal(sha(host(y)), g["cfg2_minmax/sha"])
    for size in cases.VEC_TAIL_SIZES[1:]:
        xs = x[:size + 1]
        qmax = one(4)
        y = F.min_max_quantize(dev(xs)[1:], one(-4), qmax, one(0), one(255), x_min_max=True, ema=True, decay=0.9)
        wy, wmin, wmax, _ = oracle.min_max_quantize(xs[1:], [-4], [4], [0], [255], 0.9, True, True, 0.01)
        assert np.array_equal(bits(host(y)), bits(wy))
        assert np.array_equal(bits(host(qmax)), bits(wmax))
    with pytest.raises(RuntimeError):
        F.min_max_quantize(dev(x[:64].reshape(8, 8)), dev(np.zeros((1, 4))), dev(np.ones((1, 4))),
                           dev(np.zeros((1, 4))), dev(np.ones((1, 4))))


def test_large_tensor_properties(F):
    """The headline size, 2^30 elements (4 GiB per tensor, byte offsets beyond
    2^32): idempotence of the three quantizers, their backward passes against
    masks computed from the forward's own definition, and a comparison with the
    oracle on windows at the start, across the 2^32-byte boundary and at the
    very end."""
    n = 1 << 30
    gen = torch.Generator(device="cuda").manual_seed(0)
    x = (torch.rand(n, device="cuda", generator=gen) * 9 - 4.5)
    one = lambda v: torch.tensor([v], device="cuda")
    y = F.fixed_point_quantize(x, True, 8, 2.0 ** -4)
    assert torch.equal(F.fixed_point_quantize(y, True, 8, 2.0 ** -4), y)
    p = F.pow2_quantize(x, True, True, 8, 1)
    assert torch.equal(F.pow2_quantize(p, True, True, 8, 1), p)
    qmin, qmax = one(-4.0), one(4.0)
    m = F.min_max_quantize(x, qmin, qmax, one(0.0), one(255.0))
    assert torch.equal(F.min_max_quantize(m, qmin, qmax, one(0.0), one(255.0)), m)
    W = 1 << 20
    for lo in (0, (1 << 29) - W // 2, (1 << 30) - W - 3, n - W):
        w = x[lo:lo + W].cpu().numpy()
        assert np.array_equal(bits(host(y[lo:lo + W])), bits(oracle.fixed_point_quantize(w, True, 8, 2.0 ** -4)))
        assert np.array_equal(bits(host(p[lo:lo + W])), bits(oracle.pow2_quantize(w, True, True, 8, 1)))
        assert np.array_equal(bits(host(m[lo:lo + W])), bits(oracle.min_max_quantize(w, [-4], [4], [0], [255])[0]))
    del p, m
    # backward at the same size: the gradient passes exactly where the forward did not clip
    # (step 2^-5: the clip limits +-127 * 2^-5 = +-3.97 lie inside the data range; dy := y, any tensor will do)
    dx = F.fixed_point_quantize_backward(x, y, True, 8, 2.0 ** -5, True, False)
    limit = (2.0 ** 7 - 1) * 2.0 ** -5
    inside = (x <= limit) & (x >= -limit)
    assert int((~inside).sum()) > 0
    assert torch.equal(dx, torch.where(inside, y, torch.zeros_like(y)))
    for lo in ((1 << 30) - W - 3, n - W):
        want = oracle.fixed_point_quantize_backward(x[lo:lo + W].cpu().numpy(), y[lo:lo + W].cpu().numpy(), True, 8,
                                                    2.0 ** -5)
        assert np.array_equal(bits(host(dx[lo:lo + W])), bits(want))
