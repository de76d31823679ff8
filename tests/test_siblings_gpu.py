"""GPU parity of the sibling quantization functions (BinarySigmoid, BinaryTanh,
QuantizeLinear, DequantizeLinear; forward and backward) through the C ABI,
bit-exact against the golden vectors made by the reference and against the
oracle on sizes that exercise the vector body and the tails."""
import numpy as np
import pytest
import torch

import cases
import sibling_cases
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
    def __init__(self, F):
        self.F = F

    def binary_sigmoid(self, x):
        return host(self.F.binary_sigmoid(dev(x)))

    def binary_tanh(self, x):
        return host(self.F.binary_tanh(dev(x)))

    def binary_sigmoid_backward(self, x, dy, accum, dx0):
        return host(self.F.binary_sigmoid_backward(dev(x), dev(dy), accum, dev(dx0)))

    def binary_tanh_backward(self, x, dy, accum, dx0):
        return host(self.F.binary_tanh_backward(dev(x), dev(dy), accum, dev(dx0)))

    def quantize_linear(self, x, scale, zp, mode, narrow, dtype):
        z = dev(zp)
        y = self.F.quantize_linear(dev(x), dev(scale), z, mode, narrow, dtype)
        return host(y), host(z)

    def dequantize_linear(self, x, scale, zp):
        return host(self.F.dequantize_linear(dev(x), dev(scale), dev(zp)))

    def quantize_linear_backward(self, dy, scale, accum, dx0):
        return host(self.F.quantize_linear_backward(dev(dy), dev(scale), accum, dev(dx0)))

    def dequantize_linear_backward(self, dy, scale, accum, dx0):
        return host(self.F.dequantize_linear_backward(dev(dy), dev(scale), accum, dev(dx0)))


@pytest.mark.parametrize("name", ["binary_sigmoid", "binary_tanh"])
@pytest.mark.parametrize("accum", [False, True])
def test_binary_golden(F, name, accum):
    sibling_cases.check_binary(Device(F), name, accum)


@pytest.mark.parametrize("i", range(len(cases.QL_GRID)))
def test_quantize_linear_golden(F, i):
    sibling_cases.check_quantize_linear(Device(F), i)


@pytest.mark.parametrize("i", range(len(cases.QL_SHAPES)))
@pytest.mark.parametrize("accum", [False, True])
def test_linear_rest_golden(F, i, accum):
    sibling_cases.check_linear_rest(Device(F), i, accum)


@pytest.mark.parametrize("size", [1, 5, 1023, 4099, 1 << 20])
def test_sizes_against_oracle(F, size):
    rng = np.random.RandomState(size)
    x = (rng.randn(size) * 30).astype(np.float32)
    dy = rng.randn(size).astype(np.float32)
    one = lambda v: np.array([v], np.float32)
    assert np.array_equal(bits(host(F.binary_tanh(dev(x / 30)))), bits(oracle.binary_tanh(x / 30)))
    got = F.binary_sigmoid_backward(dev(x / 30), dev(dy))
    assert np.array_equal(bits(host(got)), bits(oracle.binary_sigmoid_backward(x / 30, dy)))
    y, _ = oracle.quantize_linear(x, one(0.37), one(3.5), "HALF_TO_EVEN", False, 1)
    got = F.quantize_linear(dev(x), dev(one(0.37)), dev(one(3.5)), "HALF_TO_EVEN", False, "int8")
    assert np.array_equal(bits(host(got)), bits(y))
    got = F.dequantize_linear(dev(y), dev(one(0.37)), dev(one(4.0)))
    assert np.array_equal(bits(host(got)), bits(oracle.dequantize_linear(y, one(0.37), one(4.0))))


def test_sibling_argument_errors(F):
    x = torch.zeros(2, 3, device="cuda")
    s = torch.ones(1, 1, device="cuda")
    with pytest.raises(RuntimeError):
        F.quantize_linear(x, s, s.clone(), round_mode="NEAREST")
    with pytest.raises(RuntimeError):
        F.quantize_linear(x, s, s.clone(), dtype=5)
    with pytest.raises(RuntimeError):
        F.quantize_linear(x, torch.ones(1, device="cuda"), s.clone())
    with pytest.raises(RuntimeError):
        F.quantize_linear(x, torch.ones(2, 2, device="cuda"), s.clone())


@pytest.mark.parametrize("rate", [0.0, 0.3, 0.9, 0.999, 1.0])
@pytest.mark.parametrize("n", [1, 2, 1000, 4097, 1 << 20])
def test_prune(F, rate, n):
    rng = np.random.RandomState(n)
    x = rng.randn(n).astype(np.float32)
    x[::5] = -np.abs(x[::5])
    if n > 10:
        x[3] = x[7] = 0.0
        x[9] = -x[8]
    got = F.prune(dev(x), rate)
    assert np.array_equal(bits(host(got)), bits(oracle.prune(x, rate)))


def test_prune_special_values_and_backward(F):
    x = np.array([0.0, -0.0, 1e-45, -1e-45, 3e38, -3e38, np.inf, -np.inf, 1.0, -1.0, 0.5, 2.0], np.float32)
    for rate in (0.2, 0.5, 0.95):
        assert np.array_equal(bits(host(F.prune(dev(x), rate))), bits(oracle.prune(x, rate)))
    dy = np.arange(12, dtype=np.float32)
    dx0 = np.ones(12, np.float32)
    assert np.array_equal(host(F.prune_backward(dev(dy))), dy)
    assert np.array_equal(host(F.prune_backward(dev(dy), True, dev(dx0))), dy + 1)
    with pytest.raises(RuntimeError):
        F.prune(dev(x), 1.5)
