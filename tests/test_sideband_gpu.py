"""FixedPointQuantize that leaves int8 channel-last codes beside its fp32 result (nb200_fixed_point_quantize_nhwc_codes_f32)
and the binary-weight convolution that reads them: results identical to the plain functions, codes dropped when the
tensor changes."""
import numpy as np
import pytest
import torch

from golden_util import bits
from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def F():
    from nnabla_b200 import _capi, functions
    _capi.call("nb200_check_device")
    return functions


@pytest.fixture
def small_threshold(F):
    old = F.SIDEBAND_MIN_VALUES
    F.SIDEBAND_MIN_VALUES = 1
    yield
    F.SIDEBAND_MIN_VALUES = old


@pytest.mark.parametrize("shape,sign,n,delta", [((2, 64, 8, 8), True, 8, 2.0 ** -4), ((3, 20, 6, 10), True, 5, 0.1),
                                                ((1, 130, 4, 4), False, 7, 2.0 ** -3), ((2, 3, 2, 2), True, 8, 0.25)])
def test_quantizer_with_channel_last_codes(F, small_threshold, shape, sign, n, delta):
    rng = np.random.RandomState(sum(shape))
    x = (rng.randn(*shape) * 4).astype(np.float32)
    x.ravel()[:6] = [0.0, -0.0, 1e9, -1e9, np.float32(delta) * 2.5, -np.float32(delta) * 2.5]
    gx = torch.from_numpy(x).cuda()
    y = F.fixed_point_quantize(gx, sign, n, delta, codes_sideband=True)
    want = oracle.fixed_point_quantize(x, sign, n, delta)
    assert np.array_equal(bits(y.cpu().numpy()), bits(want))
    codes = F._sideband_get(y, delta)
    assert codes is not None and codes.dtype == torch.int8
    N, C, HW = shape[0], shape[1], shape[2] * shape[3]
    assert tuple(codes.shape) == (N, HW, F.codes_nhwc_slots(C, 1))
    k = np.rint(want.astype(np.float64) / np.float32(delta)).astype(np.int8).reshape(N, C, HW).transpose(0, 2, 1)
    got = codes.cpu().numpy()
    assert np.array_equal(got[:, :, :C], k) and not got[:, :, C:].any()
    # the plain quantizer is what runs when the conditions do not hold
    odd = torch.from_numpy(x[:, :, :1, :3].copy()).cuda()
    assert F._sideband_get(F.fixed_point_quantize(odd, sign, n, delta, codes_sideband=True), delta) is None


def test_convolution_reads_the_codes_and_stale_codes_are_dropped(F, small_threshold):
    rng = np.random.RandomState(1)
    x = torch.from_numpy((rng.randn(4, 32, 12, 12) * 3).astype(np.float32)).cuda()
    w = torch.from_numpy(rng.randn(48, 32, 3, 3).astype(np.float32)).cuda()
    wb, al = torch.zeros_like(w), torch.zeros(48, device="cuda")
    d = 2.0 ** -4
    q_plain = F.fixed_point_quantize(x, True, 8, d)
    q_codes = F.fixed_point_quantize(x, True, 8, d, codes_sideband=True)
    assert torch.equal(q_plain, q_codes)
    want = F.binary_weight_convolution(q_plain, w, wb, al, None, 1, (1, 1), (1, 1), fixed_point_delta=d)
    calls = []
    real = F.binary_weight_convolution_from_codes
    F.binary_weight_convolution_from_codes = lambda *a, **k: (calls.append(1), real(*a, **k))[1]
    try:
        got = F.binary_weight_convolution(q_codes, w, wb, al, None, 1, (1, 1), (1, 1), fixed_point_delta=d)
        assert calls == [1] and torch.equal(got, want)
        # another step, no hint, a view: the fp32 tensor is read
        F.binary_weight_convolution(q_codes, w, wb, al, None, 1, (1, 1), (1, 1), fixed_point_delta=2 * d)
        F.binary_weight_convolution(q_codes, w, wb, al, None, 1, (1, 1), (1, 1))
        F.binary_weight_convolution(q_codes.view(4, 32, 12, 12), w, wb, al, None, 1, (1, 1), (1, 1), fixed_point_delta=d)
        assert calls == [1]
        # modified through torch, or overwritten by a function of the module: the codes are gone
        q_codes.mul_(1.0)
        got = F.binary_weight_convolution(q_codes, w, wb, al, None, 1, (1, 1), (1, 1), fixed_point_delta=d)
        assert calls == [1] and torch.equal(got, want)
        q2 = F.fixed_point_quantize(x, True, 8, d, codes_sideband=True)
        F.relu(x, outputs=[q2])
        assert F._sideband_get(q2, d) is None
        n_before = len(F._sideband)
        q3 = F.fixed_point_quantize(x, True, 8, d, codes_sideband=True)
        assert len(F._sideband) == n_before + 1
        del q3
        assert len(F._sideband) == n_before  # entries go with their tensors
    finally:
        F.binary_weight_convolution_from_codes = real
    F.check_device_status()


def test_resnet18_as_written_with_the_codes_sideband(F, small_threshold):
    from nnabla_b200 import resnet18
    rng = np.random.RandomState(2)
    params = resnet18.init_parameters(rng, num_classes=16)
    gp = {k: torch.from_numpy(v).cuda() for k, v in params.items()}
    gz = lambda w, shape=None: torch.zeros(shape if shape is not None else tuple(w.shape), device="cuda")
    x = torch.from_numpy(rng.randn(2, 3, 64, 64).astype(np.float32)).cuda()
    a = resnet18.Runner(F, gp, gz)(x)
    b = resnet18.Runner(F, gp, gz, codes_sideband=True)(x)
    F.check_device_status()
    assert torch.equal(a, b)
