"""The fused BN (+ residual) + ReLU + FixedPointQuantize pass must be
bit-identical to the chain of separate functions (checked against the oracle
chain), and a ResNet-18 that uses it must produce the same logits, bit for
bit, as the unfused network on the same device."""
import numpy as np
import pytest
import torch

import cases
from oracle import ops as oracle_ops
from golden_util import bits
from oracle import oracle

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).cuda()


@pytest.fixture(scope="module")
def F():
    from nnabla_b200 import _capi, functions
    _capi.call("nb200_check_device")
    return functions


def bn_set(rng, c):
    return [(0.1 * rng.randn(c)).astype(np.float32), (1 + 0.1 * rng.randn(c)).astype(np.float32),
            (0.1 * rng.randn(c)).astype(np.float32), (0.5 + rng.rand(c)).astype(np.float32)]


@pytest.mark.parametrize("shape", [(2, 8, 6, 6), (3, 5, 7, 3), (1, 64, 56, 56), (4, 3, 1, 1)])
@pytest.mark.parametrize("second", ["none", "residual", "bn"])
@pytest.mark.parametrize("delta", [2.0 ** -4, 0.05])
def test_fused_equals_chain(F, shape, second, delta):
    rng = np.random.RandomState(sum(shape))
    a = (rng.randn(*shape) * 3).astype(np.float32)
    b = (rng.randn(*shape) * 3).astype(np.float32) if second != "none" else None
    pa = bn_set(rng, shape[1])
    pb = bn_set(rng, shape[1]) if second == "bn" else None
    want = oracle_ops.bn_add_relu_fixed_point(a, pa, b, pb, 1e-5, True, True, True, 8, delta)
    got = F.bn_add_relu_fixed_point(dev(a), [dev(t) for t in pa], dev(b) if b is not None else None,
                                    [dev(t) for t in pb] if pb else None, 1e-5, True, True, True, 8, delta)
    assert np.array_equal(bits(got.cpu().numpy()), bits(want))


def test_stages_can_be_switched_off(F):
    rng = np.random.RandomState(1)
    a = rng.randn(2, 4, 5, 5).astype(np.float32)
    pa = bn_set(rng, 4)
    want = oracle_ops.bn_add_relu_fixed_point(a, pa, None, None, 1e-5, False, False)
    got = F.bn_add_relu_fixed_point(dev(a), [dev(t) for t in pa], relu=False, quantize=False)
    assert np.array_equal(bits(got.cpu().numpy()), bits(want))
    want = oracle_ops.bn_add_relu_fixed_point(a, pa, None, None, 1e-5, True, False)
    got = F.bn_add_relu_fixed_point(dev(a), [dev(t) for t in pa], relu=True, quantize=False)
    assert np.array_equal(bits(got.cpu().numpy()), bits(want))


def test_fused_resnet_equals_unfused(F):
    from nnabla_b200 import resnet18
    rng = np.random.RandomState(0)
    params = resnet18.init_parameters(rng, num_classes=100)
    x = dev(rng.randn(2, 3, 64, 64).astype(np.float32))
    gp = {k: dev(v) for k, v in params.items()}
    gz = lambda w, shape=None: torch.zeros(shape or tuple(w.shape), device="cuda")
    plain = resnet18.Runner(F, gp, gz)(x)
    fused = resnet18.Runner(F, gp, gz, fused=True)(x)
    F.check_device_status()
    assert torch.equal(plain, fused)


# ---- activations kept as int8 channel-last codes ---------------------------------------------

def codes_of(y, delta, channels, group, slots):
    """Oracle-side layout: NCHW multiples of delta -> int8 [batch, inner, slots]."""
    n, c = y.shape[:2]
    k = np.rint(y.reshape(n, c, -1).astype(np.float64) / delta).astype(np.int64)
    assert np.abs(k).max() <= 127
    cg, pad = c // group, (c // group + 15) // 16 * 16
    out = np.zeros((n, k.shape[2], slots), np.int8)
    for g in range(group):
        out[:, :, g * pad:g * pad + cg] = k[:, g * cg:(g + 1) * cg].transpose(0, 2, 1)
    return out


@pytest.mark.parametrize("shape,group", [((2, 8, 6, 6), 1), ((3, 5, 7, 3), 1), ((1, 64, 56, 56), 1),
                                         ((2, 96, 5, 13), 1), ((2, 160, 9, 8), 1), ((2, 48, 7, 7), 3),
                                         ((1, 256, 14, 14), 1), ((4, 3, 1, 1), 1)])
@pytest.mark.parametrize("second", ["none", "residual", "bn", "codes"])
@pytest.mark.parametrize("delta", [2.0 ** -4, 0.05])
def test_fused_codes_equal_chain(F, shape, group, second, delta):
    rng = np.random.RandomState(sum(shape) + group)
    a = (rng.randn(*shape) * 3).astype(np.float32)
    pa = bn_set(rng, shape[1])
    pb = bn_set(rng, shape[1]) if second == "bn" else None
    b = b_codes = None
    slots = F.codes_nhwc_slots(shape[1], group)
    b_delta = delta * 2
    if second in ("residual", "bn"):
        b = (rng.randn(*shape) * 3).astype(np.float32)
    elif second == "codes":  # a residual that is itself a quantizer output, with its own step
        b = oracle_ops.fixed_point_quantize((rng.randn(*shape) * 3).astype(np.float32), True, 8, b_delta)
        b_codes = torch.from_numpy(codes_of(b, b_delta, shape[1], group, slots)).cuda()
    want = oracle_ops.bn_add_relu_fixed_point(a, pa, b, pb, 1e-5, True, True, True, 8, delta)
    b_dev = dev(b) if b_codes is None and b is not None else None
    got = F.bn_add_relu_fixed_point_codes(dev(a), [dev(t) for t in pa], b_dev, [dev(t) for t in pb] if pb else None,
                                          b_codes, b_delta, 1e-5, True, True, 8, delta, group)
    assert got.dtype == torch.int8 and tuple(got.shape) == (shape[0], shape[2] * shape[3], slots)
    assert np.array_equal(got.cpu().numpy(), codes_of(want, delta, shape[1], group, slots))
    # and back: code * delta is the chain's fp32 result, bit for bit
    back = F.codes_nhwc_to_float(got, shape, delta, group)
    assert np.array_equal(bits(back.cpu().numpy()), bits(want))
    # the plain re-layout of an existing quantizer output gives the same codes
    again = F.fixed_point_codes_nhwc(dev(want), delta, group)
    assert torch.equal(again, got)


@pytest.mark.parametrize("shape,group,kernel,stride,pad,ignore_border", [
    ((2, 64, 32, 32), 1, (3, 3), (2, 2), (1, 1), True),
    ((1, 20, 17, 150), 1, (3, 3), (2, 2), (1, 1), True),
    ((2, 5, 9, 11), 1, (2, 2), (2, 2), (0, 0), True),
    ((2, 33, 10, 13), 1, (3, 2), (1, 2), (1, 0), False),
    ((1, 48, 12, 12), 3, (3, 3), (2, 2), (1, 1), False),
    ((1, 160, 7, 7), 1, (7, 7), (1, 1), (0, 0), True),
])
def test_max_pooling_on_codes_equals_chain(F, shape, group, kernel, stride, pad, ignore_border):
    rng = np.random.RandomState(sum(shape))
    delta = 2.0 ** -4
    q = oracle_ops.fixed_point_quantize((rng.randn(*shape) * 3).astype(np.float32), True, 8, delta)
    want = oracle_ops.max_pooling(q, kernel, stride, ignore_border, pad)
    slots = F.codes_nhwc_slots(shape[1], group)
    codes = F.fixed_point_codes_nhwc(dev(q), delta, group)
    got, pooled = F.max_pooling_codes(codes, shape, kernel, stride, ignore_border, pad, group)
    assert tuple(pooled) == tuple(want.shape)
    assert np.array_equal(got.cpu().numpy(), codes_of(want, delta, shape[1], group, slots))


def test_fused_codes_without_relu_and_unsigned(F):
    rng = np.random.RandomState(3)
    shape = (2, 20, 6, 10)
    a = (rng.randn(*shape) * 3).astype(np.float32)
    pa = bn_set(rng, shape[1])
    slots = F.codes_nhwc_slots(shape[1], 1)
    for relu, sign, n in ((False, True, 8), (False, True, 4), (True, False, 7), (False, False, 5)):
        want = oracle_ops.bn_add_relu_fixed_point(a, pa, None, None, 1e-5, relu, True, sign, n, 0.125)
        got = F.bn_add_relu_fixed_point_codes(dev(a), [dev(t) for t in pa], relu=relu, sign=sign, n=n, delta=0.125)
        assert np.array_equal(got.cpu().numpy(), codes_of(want, 0.125, shape[1], 1, slots)), (relu, sign, n)
    from nnabla_b200._capi import NB200Error
    with pytest.raises(NB200Error):  # 8 unsigned bits do not fit an int8 code
        F.bn_add_relu_fixed_point_codes(dev(a), [dev(t) for t in pa], sign=False, n=8)


@pytest.mark.parametrize("case", [
    dict(x=(2, 64, 14, 14), ko=64, k=3, pad=1, stride=1, group=1),
    dict(x=(3, 128, 9, 9), ko=256, k=3, pad=1, stride=2, group=1),
    dict(x=(2, 48, 8, 8), ko=24, k=1, pad=0, stride=2, group=3),
    dict(x=(1, 20, 12, 10), ko=40, k=3, pad=1, stride=1, group=1),
])
def test_convolution_from_codes_equals_hinted_convolution(F, case):
    rng = np.random.RandomState(case["ko"])
    delta = 2.0 ** -4
    xs, ko, k, g = case["x"], case["ko"], case["k"], case["group"]
    xq = oracle_ops.fixed_point_quantize(np.maximum(rng.randn(*xs), 0).astype(np.float32) * 2, True, 8, delta)
    w = (rng.randn(ko, xs[1] // g, k, k) * 0.1).astype(np.float32)
    bias = (0.1 * rng.randn(ko)).astype(np.float32)
    gz = lambda *s: torch.zeros(*s, device="cuda")
    pad, stride = (case["pad"],) * 2, (case["stride"],) * 2
    wb1, al1 = gz(*w.shape), gz(ko)
    want = F.binary_weight_convolution(dev(xq), dev(w), wb1, al1, dev(bias), 1, pad, stride, (1, 1), g, 1.0,
                                       fixed_point_delta=delta)
    codes = F.fixed_point_codes_nhwc(dev(xq), delta, g)
    wb2, al2 = gz(*w.shape), gz(ko)
    got = F.binary_weight_convolution_from_codes(codes, xs, dev(w), wb2, al2, dev(bias), pad, stride, (1, 1), g, 1.0,
                                                 delta)
    F.check_device_status()
    assert torch.equal(got, want) and torch.equal(wb1, wb2) and torch.equal(al1, al2)
    # and against the oracle directly: signs bit-exact, outputs within 1e-5 of the output RMS
    oy, owb, _ = oracle.binary_weight_convolution(xq, w, bias, pad, stride, (1, 1), g, 1.0)
    assert np.array_equal(bits(wb2.cpu().numpy()), bits(owb))
    assert cases.rel_rms(got.cpu().numpy(), oy) < 1e-5
    # binary connect: no alpha
    wb3 = gz(*w.shape)
    want_c = F.binary_connect_convolution(dev(xq), dev(w), wb3, None, 1, pad, stride, (1, 1), g, 1.0,
                                          fixed_point_delta=delta)
    got_c = F.binary_weight_convolution_from_codes(codes, xs, dev(w), gz(*w.shape), None, None, pad, stride, (1, 1), g,
                                                   1.0, delta)
    assert torch.equal(got_c, want_c)


def test_prepared_weights_equal_per_call_binarisation(F):
    rng = np.random.RandomState(21)
    delta = 2.0 ** -4
    for xs, ko, k, g, stride in (((2, 64, 14, 14), 64, 3, 1, 1), ((2, 48, 9, 9), 24, 3, 3, 2), ((1, 160, 8, 8), 200, 1, 1, 1)):
        xq = oracle_ops.fixed_point_quantize(np.maximum(rng.randn(*xs), 0).astype(np.float32) * 2, True, 8, delta)
        w = (rng.randn(ko, xs[1] // g, k, k) * 0.1).astype(np.float32)
        w[0, 0, 0, 0] = 0.0
        bias = (0.1 * rng.randn(ko)).astype(np.float32)
        codes = F.fixed_point_codes_nhwc(dev(xq), delta, g)
        pad, st = (k // 2, k // 2), (stride, stride)
        wb = torch.zeros(*w.shape, device="cuda")
        al = torch.zeros(ko, device="cuda")
        want = F.binary_weight_convolution_from_codes(codes, xs, dev(w), wb, al, dev(bias), pad, st, (1, 1), g, 1.0, delta)
        prep = F.prepare_binary_weights(dev(w), g, 1.0)
        got = F.binary_convolution_from_codes_prepared(codes, xs, prep, dev(bias), pad, st, (1, 1), delta)
        F.check_device_status()
        assert torch.equal(got, want) and torch.equal(prep.binary_weight, wb) and torch.equal(prep.alpha, al)
        oy, owb, oal = oracle.binary_weight_convolution(xq, w, bias, pad, st, (1, 1), g, 1.0)
        assert np.array_equal(bits(prep.binary_weight.cpu().numpy()), bits(owb))
        np.testing.assert_allclose(prep.alpha.cpu().numpy(), np.abs(w.astype(np.float64)).reshape(ko, -1).mean(1),
                                   rtol=1e-6)
        np.testing.assert_allclose(prep.alpha.cpu().numpy(), oal, rtol=1e-5)
        assert cases.rel_rms(got.cpu().numpy(), oy) < 1e-5
        # BinaryConnect: no alpha
        wbc = torch.zeros(*w.shape, device="cuda")
        want_c = F.binary_weight_convolution_from_codes(codes, xs, dev(w), wbc, None, None, pad, st, (1, 1), g, 1.0, delta)
        prep_c = F.prepare_binary_weights(dev(w), g, 1.0, with_alpha=False)
        assert torch.equal(F.binary_convolution_from_codes_prepared(codes, xs, prep_c, None, pad, st, (1, 1), delta), want_c)


def test_codes_resnet_equals_unfused(F):
    from nnabla_b200 import resnet18
    rng = np.random.RandomState(0)
    params = resnet18.init_parameters(rng, num_classes=100)
    x = dev(rng.randn(3, 3, 96, 64).astype(np.float32))
    gp = {k: dev(v) for k, v in params.items()}
    gz = lambda w, shape=None: torch.zeros(shape or tuple(w.shape), device="cuda")
    plain = resnet18.Runner(F, gp, gz)(x)
    codes = resnet18.Runner(F, gp, gz, fused="codes")(x)
    F.check_device_status()
    assert torch.equal(plain, codes)
    net = resnet18.Runner(F, gp, gz, fused="codes", prepared_weights=True)
    assert torch.equal(plain, net(x)) and torch.equal(plain, net(x))  # first call prepares, second reuses
    F.check_device_status()


def test_normalisation_with_extreme_statistics(F):
    """Zeros of both signs, denormal-range and huge inputs, infinities and tiny / huge variances
    go through the same rounded operations as the reference's (NaN positions must agree)."""
    rng = np.random.RandomState(9)
    shape = (2, 12, 4, 8)
    a = (rng.randn(*shape) * 3).astype(np.float32)
    a[0, 0] = 0.0
    a[0, 1] = -0.0
    a[1, 2] *= 1e-35
    a[1, 3] *= 1e30
    a[0, 4, 0, 0] = np.inf
    a[0, 5, 0, 0] = np.nan
    pa = bn_set(rng, shape[1])
    pa[3][6:9] = [1e-30, 1e30, 3e-13]  # variance
    pa[2][0:2] = 0.0                   # mean, so that zeros stay zeros
    pa[0][0] = -0.0
    want = oracle_ops.bn_add_relu_fixed_point(a, pa, None, None, 1e-5, False, False)

    def same(got):
        got = got.cpu().numpy()
        nan = np.isnan(want)
        return np.array_equal(np.isnan(got), nan) and np.array_equal(bits(got)[~nan], bits(want)[~nan])
    assert same(F.bn_add_relu_fixed_point(dev(a), [dev(t) for t in pa], relu=False, quantize=False))
    assert same(F.batch_normalization(dev(a), *[dev(t) for t in pa], axes=[1], eps=1e-5, batch_stat=False))


def test_forward_captured_as_cuda_graph(F):
    """The library's calls are stream-ordered, so a whole forward can be recorded into a CUDA graph
    and replayed: same logits, also for new inputs."""
    from nnabla_b200 import graphs, resnet18
    rng = np.random.RandomState(5)
    params = resnet18.init_parameters(rng, num_classes=100)
    gp = {k: dev(v) for k, v in params.items()}
    gz = lambda w, shape=None: torch.zeros(shape or tuple(w.shape), device="cuda")
    x = dev(rng.randn(2, 3, 64, 64).astype(np.float32))
    net = resnet18.Runner(F, gp, gz, fused="codes", prepared_weights=True)
    want = net(x).clone()
    captured = graphs.Captured(net, x)
    assert torch.equal(captured(x), want)
    x2 = dev(rng.randn(2, 3, 64, 64).astype(np.float32))
    assert torch.equal(captured(x2), net(x2))
    assert torch.equal(captured(x), want)
    F.check_device_status()
