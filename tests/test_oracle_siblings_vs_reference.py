"""Pins the C restatement of the sibling quantization functions
(oracle/oracle_siblings.c) bit for bit against the reference's own compiled
CPU functions (oracle/_ref/libnnabla_ref.so), forward and backward."""
import numpy as np
import pytest

import cases
from oracle import oracle, ref

pytestmark = pytest.mark.skipif(not ref.available(), reason="reference CPU library not built")


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


@pytest.mark.parametrize("name", ["binary_sigmoid", "binary_tanh"])
@pytest.mark.parametrize("accum", [False, True])
def test_binary_activations(name, accum):
    x = cases.binary_act_input()
    dy, dx0 = cases.grad_inputs(x)
    assert np.array_equal(bits(getattr(oracle, name)(x)), bits(getattr(ref, name)(x)))
    want = getattr(ref, name + "_backward")(x, dy, accum, dx0)
    got = getattr(oracle, name + "_backward")(x, dy, accum, dx0)
    assert np.array_equal(bits(got), bits(want))


@pytest.mark.parametrize("shapes,round_mode,narrow,dtype", cases.QL_GRID)
def test_quantize_linear(shapes, round_mode, narrow, dtype):
    x, scale, zp = cases.quantize_linear_inputs(*shapes)
    wy, wzp = ref.quantize_linear(x, scale, zp, round_mode, narrow, dtype)
    gy, gzp = oracle.quantize_linear(x, scale, zp, round_mode, narrow, dtype)
    assert np.array_equal(bits(gzp), bits(wzp))
    assert np.array_equal(bits(gy), bits(wy))


@pytest.mark.parametrize("shapes", cases.QL_SHAPES)
@pytest.mark.parametrize("accum", [False, True])
def test_linear_backward_and_dequantize(shapes, accum):
    x, scale, zp = cases.quantize_linear_inputs(*shapes)
    dy, dx0 = cases.grad_inputs(x)
    assert np.array_equal(bits(oracle.dequantize_linear(x, scale, zp)), bits(ref.dequantize_linear(x, scale, zp)))
    want = ref.quantize_linear_backward(x, scale, zp, dy, accum=accum, dx=dx0)
    assert np.array_equal(bits(oracle.quantize_linear_backward(dy, scale, accum, dx0)), bits(want))
    want = ref.dequantize_linear_backward(x, scale, zp, dy, accum=accum, dx=dx0)
    assert np.array_equal(bits(oracle.dequantize_linear_backward(dy, scale, accum, dx0)), bits(want))


@pytest.mark.parametrize("rate", [0.0, 0.3, 0.9, 0.999, 1.0])
@pytest.mark.parametrize("n", [1, 2, 1000, 4097])
def test_prune(rate, n):
    rng = np.random.RandomState(n)
    x = rng.randn(n).astype(np.float32)
    x[::5] = -np.abs(x[::5])
    if n > 10:
        x[3] = x[7] = 0.0          # ties and zeros
        x[9] = -x[8]
    assert np.array_equal(bits(oracle.prune(x, rate)), bits(ref.prune(x, rate)))
