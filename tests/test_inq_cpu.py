"""The C restatement of INQAffine's weight update (oracle/oracle_inq.c) against the reference's own compiled
function, over several forward passes of one function instance (the state machine advances)."""
import numpy as np
import pytest

import inq_cases
from oracle import oracle, ref

pytestmark = pytest.mark.skipif(not ref.available(), reason="oracle/_ref (reference build) not present")


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


@pytest.mark.parametrize("i", range(len(inq_cases.CASES)))
def test_inq_affine_largest_abs(i):
    x, w, ind, b, nbits, its, passes = inq_cases.inputs(i)
    outs, ins, _ = ref.forward("INQAffine", [1, nbits, 0, 7], [its], [x, w, ind, b], repeat=passes)
    st = oracle.INQState(w.shape)
    ww, ii = w, ind.astype(np.int32)
    for _ in range(passes):
        y, ww, ii = oracle.inq_affine(x, ww, ii, b, st, 1, nbits, its)
    assert np.array_equal(bits(ins[1]), bits(ww))
    assert np.array_equal(ins[2].astype(np.int32), ii)
    assert np.allclose(outs[0], y, rtol=1e-5, atol=1e-5)
    fixed = ii == 1
    if fixed.any():  # fixed weights are zero or signed powers of two
        m = np.abs(ww[fixed])
        nz = m[m > 0]
        assert np.array_equal(np.exp2(np.round(np.log2(nz))), nz)


@pytest.mark.parametrize("i", range(len(inq_cases.CONV_CASES)))
def test_inq_convolution_largest_abs(i):
    x, w, ind, b, pad, stride, dilation, group, nbits, its, passes = inq_cases.conv_inputs(i)
    outs, ins, _ = ref.forward("INQConvolution", [1, group, nbits, 0, 7], [list(pad), list(stride), list(dilation), its],
                               [x, w, ind, b], repeat=passes)
    st = oracle.INQState(w.shape)
    ww, ii = w, ind.astype(np.int32)
    for _ in range(passes):
        y, ww, ii = oracle.inq_convolution(x, ww, ii, b, st, pad, stride, dilation, group, nbits, its)
    assert np.array_equal(bits(ins[1]), bits(ww))
    assert np.array_equal(ins[2].astype(np.int32), ii)
    assert np.allclose(outs[0], y, rtol=1e-4, atol=1e-4 * float(np.abs(y).max()))


def test_exponent_rule_is_one_step_per_binade():
    """floor(log2 a) + (log2 a - floor >= log2 1.5) with a float logarithm: inside every binade the result is e
    below some mantissa and e + 1 from it on (where exactly depends on how log2f rounds at that magnitude,
    which is why the CUDA side tabulates the step per binade from the host libm)."""
    import ctypes
    L = oracle.lib()
    rng = np.random.RandomState(0)
    for e in range(-140, 127, 7):
        m = np.sort(rng.uniform(1.0, 2.0, size=200))
        vals = [L.oracle_inq_exponent(ctypes.c_float(float(np.float32(v * 2.0 ** e)))) for v in m]
        assert set(vals) <= {e, e + 1} and vals == sorted(vals)
        assert vals[0] == e and vals[-1] == e + 1
