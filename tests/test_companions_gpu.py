"""GPU parity of the companion functions (BN inference, ReLU, Add2, max
pooling, global average pooling, full-precision stem convolution): bit-exact
against the oracle, which is itself bit-exact against the reference's CPU code."""
import numpy as np
import pytest
import torch

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


# planes of 1 value (per-value kernel), 32 .. 1023 values (a warp per plane: float4 lanes when the plane is a
# multiple of 4 values, scalar lanes otherwise, with and without the loop past the first four loads), 1024 and more
# (a block per plane)
@pytest.mark.parametrize("shape", [(2, 6, 9, 11), (3, 16, 8, 8), (1, 5, 1, 1), (4, 7), (2, 5, 7, 7), (2, 3, 28, 28),
                                   (3, 4, 20, 10), (2, 3, 13, 31), (2, 2, 4, 8), (1, 3, 31, 33), (1, 2, 32, 32),
                                   (9, 3, 5, 6), (2, 3, 48, 48), (4, 8, 7, 7), (2, 6, 13, 31), (2, 2, 5, 7), (1, 4, 11, 93)])
def test_batch_normalization_relu_add2(F, shape):
    rng = np.random.RandomState(sum(shape))
    x = rng.randn(*shape).astype(np.float32)
    C = shape[1]
    pshape = (1, C) + (1,) * (len(shape) - 2)
    beta, gamma, mean = (rng.randn(*pshape).astype(np.float32) for _ in range(3))
    var = (rng.rand(*pshape) + 0.1).astype(np.float32)
    y = F.batch_normalization(dev(x), dev(beta), dev(gamma), dev(mean), dev(var), [1], 0.9, 1e-5, False)
    x3 = x.reshape(shape[0], C, -1)
    assert np.array_equal(bits(host(y)).reshape(-1), bits(oracle.batch_norm_inference(x3, beta, gamma, mean, var, 1e-5)).reshape(-1))
    assert np.array_equal(bits(host(F.relu(dev(x)))), bits(oracle.relu(x)))
    x2 = rng.randn(*shape).astype(np.float32)
    assert np.array_equal(bits(host(F.add2(dev(x), dev(x2)))), bits(oracle.add2(x, x2)))


@pytest.mark.parametrize("k,s,p,ib", [((3, 3), (2, 2), (1, 1), True), ((2, 2), (2, 2), (0, 0), True),
                                      ((3, 3), (2, 2), (0, 0), False), ((3, 2), (1, 2), (1, 0), True)])
def test_pooling(F, k, s, p, ib):
    rng = np.random.RandomState(7)
    x = rng.randn(2, 5, 13, 10).astype(np.float32)
    assert np.array_equal(bits(host(F.max_pooling(dev(x), k, s, ib, p))), bits(oracle.max_pooling(x, k, s, ib, p)))
    assert np.array_equal(bits(host(F.global_average_pooling(dev(x)))), bits(oracle.global_average_pooling(x)))


@pytest.mark.parametrize("xs,ws,pad,stride", [((2, 3, 32, 32), (64, 3, 7, 7), (3, 3), (2, 2)),
                                              ((2, 3, 56, 56), (64, 3, 7, 7), (3, 3), (2, 2)),   # band kernel, one band
                                              ((1, 3, 224, 224), (64, 3, 7, 7), (3, 3), (2, 2)),  # band kernel, 7 bands
                                              ((2, 2, 30, 28), (20, 2, 5, 7), (2, 3), (3, 2)),    # ragged maps and rows
                                              ((1, 3, 27, 29), (8, 3, 7, 7), (3, 1), (2, 2)),     # 7 does not divide Wo

                                              ((3, 3, 224, 224), (64, 3, 7, 7), (3, 3), (2, 2)),  # tensor cores, 3 tiles per SM
                                              ((2, 1, 64, 100), (48, 1, 6, 24), (2, 11), (2, 2)), # one channel, 24-wide filter rows
                                              ((2, 4, 40, 36), (64, 4, 3, 5), (1, 2), (1, 1)),    # 4 channels, stride 1
                                              ((1, 3, 17, 19), (20, 3, 3, 3), (1, 1), (1, 1)),
                                              ((2, 4, 9, 9), (5, 4, 1, 1), (0, 0), (2, 2))])
def test_full_precision_convolution(F, xs, ws, pad, stride):
    rng = np.random.RandomState(11)
    x = rng.randn(*xs).astype(np.float32)
    w = rng.randn(*ws).astype(np.float32)
    b = rng.randn(ws[0]).astype(np.float32)
    y = host(F.convolution(dev(x), dev(w), dev(b), 1, pad, stride))
    want = oracle.convolution(x, w, b, pad, stride)
    assert y.shape == want.shape
    # fp32 rounding differs from the oracle's separate mul / add: fused multiply-adds in the CUDA-core
    # kernel (about 1e-7), truncating fp32 accumulation of bf16 piece products on the tensor cores
    # (about 6e-7 of the output RMS); the bar for contractions is 1e-5 of the output RMS
    assert cases.rel_rms(y, want) < 2e-6


@pytest.mark.parametrize("xs,ws,pad,stride", [((1, 3, 20, 256), (64, 3, 7, 7), (3, 3), (2, 2)),   # 128 output columns: every MMA row
                                              ((2, 8, 12, 128), (40, 8, 3, 3), (1, 1), (1, 1)),   # 8 channels at stride 1, 128 columns
                                              ((2, 1, 33, 41), (7, 1, 8, 4), (4, 1), (1, 2)),     # 8 filter rows, one channel
                                              ((5, 3, 32, 32), (64, 3, 7, 7), (3, 3), (2, 2))])
def test_stem_convolution_edges(F, xs, ws, pad, stride):
    """Geometries at the limits of the tensor-core stem kernel, and inputs that exercise its per-sample
    scaling: samples of very different magnitude in one batch, a sample of zeros, tiny and large weights."""
    rng = np.random.RandomState(sum(xs))
    x = rng.randn(*xs).astype(np.float32)
    w = rng.randn(*ws).astype(np.float32)
    b = rng.randn(ws[0]).astype(np.float32)
    scales = [1.0, 3e4, 1e-5, 0.0, 7.0][:xs[0]]
    for n, sc in enumerate(scales):
        x[n] *= np.float32(sc)
    for wscale in (1.0, 1e-4, 2e3):
        ww = (w * np.float32(wscale)).astype(np.float32)
        y = host(F.convolution(dev(x), dev(ww), dev(b), 1, pad, stride))
        F.check_device_status()
        want = oracle.convolution(x, ww, None, pad, stride)
        for n in range(xs[0]):  # every sample against its own magnitude
            if scales[n] == 0.0:
                assert np.array_equal(y[n], np.broadcast_to(b.reshape(-1, 1, 1), y[n].shape))
                continue
            rms = np.sqrt(np.mean(want[n].astype(np.float64) ** 2))
            err = np.sqrt(np.mean((y[n].astype(np.float64) - (want[n].astype(np.float64) + b.reshape(-1, 1, 1))) ** 2))
            # the bias addition rounds at the size of max(|conv|, |bias|)
            assert err <= 2e-6 * rms + 1.2e-7 * (np.abs(b).max() + np.abs(want[n]).max()), (n, wscale, err, rms)


@pytest.mark.parametrize("shape", [(2, 3, 16, 16), (1, 4, 13, 24), (3, 2, 8, 8), (1, 1, 56, 112)])
@pytest.mark.parametrize("ib", [True, False])
def test_pooling_3x3_stride2_vector_path(F, shape, ib):
    """Widths that take the four-outputs-per-thread kernel; zeros of both signs
    and repeated values make the first-maximum-wins rule visible."""
    rng = np.random.RandomState(sum(shape))
    x = rng.randn(*shape).astype(np.float32)
    x[rng.rand(*shape) < 0.3] = 0.0
    x[rng.rand(*shape) < 0.2] = -0.0
    x = np.minimum(x, 0.0) if shape[0] == 3 else x          # all windows hold only zeros and negatives
    got = F.max_pooling(dev(x), (3, 3), (2, 2), ib, (1, 1))
    assert np.array_equal(bits(host(got)), bits(oracle.max_pooling(x, (3, 3), (2, 2), ib, (1, 1))))


def test_batch_normalization_division_is_ieee_exact_over_wide_ranges(F):
    """The normalisation's quotient must be the IEEE fp32 quotient for every magnitude, down to subnormal
    results, whatever way the kernel takes to divide by its per-channel constant."""
    rng = np.random.RandomState(21)
    C, S = 96, 4096
    mag = np.exp(rng.uniform(np.log(1e-38), np.log(1e38), size=(8, C, S))).astype(np.float32)
    x = (mag * rng.choice([-1.0, 1.0], size=mag.shape)).astype(np.float32)
    x[0, :, :64] = 0.0
    x[1, :, :64] = -0.0
    x[2, :, :256] = rng.randint(-2 ** 23, 2 ** 23, size=(C, 256)).astype(np.float32) * np.float32(2.0 ** -149)  # subnormals
    x[3, :, :256] = rng.randint(1, 2 ** 24, size=(C, 256)).astype(np.float32)                              # integers
    var = np.exp(rng.uniform(np.log(1e-12), np.log(1e12), size=C)).astype(np.float32)
    var[:8] = np.float32([4.0, 0.25, 1.0, 9.0, 2.0 ** 40, 2.0 ** -40, 3.0, 1e-30]) - np.float32(1e-5)  # exact roots, tiny
    var = np.maximum(var, np.float32(0.0))
    gamma = np.ones(C, np.float32)
    gamma[::3] = np.exp(rng.uniform(-20, 20, size=len(gamma[::3]))).astype(np.float32)
    beta = np.zeros(C, np.float32)
    mean = np.zeros(C, np.float32)
    mean[1::2] = rng.randn(len(mean[1::2])).astype(np.float32)
    with np.errstate(all="ignore"):
        want = oracle.batch_norm_inference(x, beta, gamma, mean, var, 1e-5)
    got = host(F.batch_normalization(dev(x), dev(beta), dev(gamma), dev(mean), dev(var), [1], 0.9, 1e-5, False))
    assert np.array_equal(bits(got).reshape(-1), bits(want).reshape(-1))
