"""INQAffine / INQConvolution on the GPU: the C-ABI weight update (nb200_inq_restore_f32 / nb200_inq_quantize_f32 through
nnabla_b200.functions.inq_affine) against the oracle over several forward passes, and the extension class
against nnabla's own CPU function through Function::forward (largest-magnitude and random selection)."""
import numpy as np
import pytest
import torch

import ext_harness as H
import inq_cases
from golden_util import bits
from oracle import oracle

pytestmark = pytest.mark.gpu


def dev(a, dtype=np.float32):
    return torch.from_numpy(np.ascontiguousarray(a, dtype)).cuda()


def close_to_rms(got, want, tol=1e-5):
    """The contraction's tolerance: every output within tol of the output RMS (fp32 summation order differs)."""
    rms = float(np.sqrt(np.mean(np.square(want.astype(np.float64))))) + 1e-30
    return float(np.max(np.abs(got.astype(np.float64) - want))) <= tol * rms


@pytest.fixture(scope="module")
def F():
    from nnabla_b200 import _capi, functions
    _capi.call("nb200_check_device")
    return functions


@pytest.mark.parametrize("i", range(len(inq_cases.CASES)))
def test_inq_affine_mirror_against_oracle(F, i):
    x, w, ind, b, nbits, its, passes = inq_cases.inputs(i)
    st = oracle.INQState(w.shape)
    ww, ii = w, ind.astype(np.int32)
    gw, gi = dev(w), dev(ind, np.int32)
    gst = F.INQState(gw)
    for _ in range(passes):
        y, ww, ii = oracle.inq_affine(x, ww, ii, b, st, 1, nbits, its)
        gy = F.inq_affine(dev(x), gw, gi, dev(b), 1, nbits, its, "largest_abs", -1, gst)
        F.check_device_status()
        assert np.array_equal(bits(gw.cpu().numpy()), bits(ww))
        assert np.array_equal(gi.cpu().numpy(), ii)
        assert np.array_equal(bits(gst.old_weights.cpu().numpy()), bits(st.old_w))
        assert np.array_equal(gst.old_indicators.cpu().numpy(), st.old_ind)
        assert close_to_rms(gy.cpu().numpy(), y)


def test_inq_quantize_edge_values(F):
    """Zeros of both signs, denormals, values at and around 1.5 * 2^e and the window's ends, all fixed."""
    rng = np.random.RandomState(1)
    vals = [0.0, -0.0, 1e-45, -3e-42, 1.17e-38, 0.375, -0.375, 1.5, 3.0, 96.0, 100.0, -127.9, 2.0 ** -30, 7e-5]
    for e in (-20, -3, 0, 5):
        a = np.float32(1.5 * 2.0 ** e)
        for _ in range(3):
            vals += [float(a), -float(np.nextafter(a, np.float32(np.inf))), float(np.nextafter(a, np.float32(-np.inf)))]
            a = np.nextafter(a, np.float32(np.inf))
    w = np.array(vals + list(rng.randn(200) * np.exp(rng.uniform(-30, 4, size=200))), np.float32).reshape(1, -1)
    for nbits in (2, 3, 4, 6, 8):
        st = oracle.INQState(w.shape)
        ww, ii = oracle.inq_update(w, np.zeros(w.shape, np.int32), st, nbits, [0])
        gw, gi = dev(w), dev(np.zeros(w.shape), np.int32)
        gst = F.INQState(gw)
        F.inq_update_weights(gw, gi, gst, nbits, [0])
        assert np.array_equal(bits(gw.cpu().numpy()), bits(ww)), nbits
        assert np.array_equal(gi.cpu().numpy(), ii)


@pytest.mark.parametrize("i", range(len(inq_cases.CASES)))
@pytest.mark.parametrize("algorithm", [0, 1])
def test_inq_affine_extension_against_cpu_context(i, algorithm):
    x, w, ind, b, nbits, its, passes = inq_cases.inputs(i)
    args = ("INQAffine", [1, nbits, algorithm, 11 + i], [its], [x, w, ind, b])
    c = H.forward("cpu:float", *args, repeat=passes)
    g = H.forward("b200:float", *args, repeat=passes)
    assert c[2] == g[2] == "INQAffine"
    assert np.array_equal(bits(g[1][1]), bits(c[1][1]))        # weights after
    assert np.array_equal(g[1][2], c[1][2])                    # indicators after
    assert close_to_rms(g[0][0], c[0][0])


@pytest.mark.parametrize("i", range(len(inq_cases.CONV_CASES)))
def test_inq_convolution_mirror_against_oracle(F, i):
    x, w, ind, b, pad, stride, dilation, group, nbits, its, passes = inq_cases.conv_inputs(i)
    st = oracle.INQState(w.shape)
    ww, ii = w, ind.astype(np.int32)
    gw, gi = dev(w), dev(ind, np.int32)
    gst = F.INQState(gw)
    for _ in range(passes):
        y, ww, ii = oracle.inq_convolution(x, ww, ii, b, st, pad, stride, dilation, group, nbits, its)
        gy = F.inq_convolution(dev(x), gw, gi, dev(b), 1, pad, stride, dilation, group, nbits, its, "largest_abs", -1,
                               gst)
        F.check_device_status()
        assert np.array_equal(bits(gw.cpu().numpy()), bits(ww))
        assert np.array_equal(gi.cpu().numpy(), ii)
        assert close_to_rms(gy.cpu().numpy(), y)


@pytest.mark.parametrize("i", range(len(inq_cases.CONV_CASES)))
@pytest.mark.parametrize("algorithm", [0, 1])
def test_inq_convolution_extension_against_cpu_context(i, algorithm):
    x, w, ind, b, pad, stride, dilation, group, nbits, its, passes = inq_cases.conv_inputs(i)
    args = ("INQConvolution", [1, group, nbits, algorithm, 5 + i], [list(pad), list(stride), list(dilation), its],
            [x, w, ind, b])
    c = H.forward("cpu:float", *args, repeat=passes)
    g = H.forward("b200:float", *args, repeat=passes)
    assert c[2] == g[2] == "INQConvolution"
    assert np.array_equal(bits(g[1][1]), bits(c[1][1]))
    assert np.array_equal(g[1][2], c[1][2])
    assert close_to_rms(g[0][0], c[0][0])


def test_inq_backward_goes_through_the_inner_function():
    """INQAffine / INQConvolution::backward_impl hand the gradients to the inner Affine / Convolution
    (inq_affine.cpp:218-232, inq_convolution.cpp:222-237), which under this context are the device ones."""
    import cases
    x, w, ind, b, nbits, its, _ = inq_cases.inputs(3)
    rng = np.random.RandomState(3)
    gy = rng.randn(x.shape[0], w.shape[1]).astype(np.float32)
    g0 = [rng.randn(*a.shape).astype(np.float32) for a in (x, w, ind, b)]
    for accum in (False, True):
        args = ("INQAffine", [1, nbits, 0, 3], [its], [x, w, ind, b], [gy], [True, True, False, True], [accum] * 4, g0)
        c, g = H.backward("cpu:float", *args), H.backward("b200:float", *args)
        for k in (0, 1, 3):
            assert cases.rel_rms(g[0][k], c[0][k]) < 1e-5, (accum, k)
    x, w, ind, b, pad, stride, dilation, group, nbits, its, _ = inq_cases.conv_inputs(0)
    y_shape = oracle.conv_out_shape(x.shape, w.shape, pad, stride, dilation)
    gy = rng.randn(*y_shape).astype(np.float32)
    g0 = [rng.randn(*a.shape).astype(np.float32) for a in (x, w, ind, b)]
    for accum in (False, True):
        args = ("INQConvolution", [1, group, nbits, 0, 3], [list(pad), list(stride), list(dilation), its],
                [x, w, ind, b], [gy], [True, True, False, True], [accum] * 4, g0)
        c, g = H.backward("cpu:float", *args), H.backward("b200:float", *args)
        for k in (0, 1, 3):
            assert cases.rel_rms(g[0][k], c[0][k]) < 1e-5, (accum, k)


def test_parametric_inq_layers(F):
    """PF.inq_affine / PF.inq_convolution (parametric_functions.py:493, :1126): parameters W, I, b under the
    scopes "inq_affine" / "inq_conv", the function's state kept with the layer across calls."""
    from nnabla_b200 import parametric_functions as PF
    PF.clear_parameters()
    x, w, ind, b, nbits, its, passes = inq_cases.inputs(3)
    st = oracle.INQState(w.shape)
    ww, ii = w, ind.astype(np.int32)
    for _ in range(passes):
        y, ww, ii = oracle.inq_affine(x, ww, ii, b, st, 1, nbits, its)
        with PF.parameter_scope("fc"):
            gy = PF.inq_affine(dev(x), w.shape[1], 1, nbits, its, "largest_abs", w_init=w, b_init=b)
        params = PF.get_parameters()
        assert np.array_equal(bits(params["fc/inq_affine/W"].cpu().numpy()), bits(ww))
        assert np.array_equal(params["fc/inq_affine/I"].cpu().numpy(), ii)
        assert close_to_rms(gy.cpu().numpy(), y)
    x, w, ind, b, pad, stride, dilation, group, nbits, its, passes = inq_cases.conv_inputs(0)
    st = oracle.INQState(w.shape)
    ww, ii = w, ind.astype(np.int32)
    for _ in range(passes):
        y, ww, ii = oracle.inq_convolution(x, ww, ii, b, st, pad, stride, dilation, group, nbits, its)
        with PF.parameter_scope("c1"):
            gy = PF.inq_convolution(dev(x), w.shape[0], w.shape[2:], pad, stride, dilation, group, nbits, its,
                                    "largest_abs", w_init=w, b_init=b)
        params = PF.get_parameters()
        assert np.array_equal(bits(params["c1/inq_conv/W"].cpu().numpy()), bits(ww))
        assert np.array_equal(params["c1/inq_conv/I"].cpu().numpy(), ii)
        assert close_to_rms(gy.cpu().numpy(), y)
    PF.clear_parameters()
