"""GPU parity of the binary convolutions' backward passes through the C ABI
against the oracle: dx, dW and db within 1e-5 of their RMS (the tolerance
stated for convolution outputs), judged against the float64 sums as well."""
import numpy as np
import pytest
import torch

import cases
from oracle import oracle

pytestmark = pytest.mark.gpu
TOL = 1e-5


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).cuda()


@pytest.fixture(scope="module")
def F():
    from nnabla_b200 import _capi, functions
    _capi.call("nb200_check_device")
    return functions


# (x shape, w shape, pad, stride, dilation, group)
BACKWARD_CASES = cases.CONV_CASES + [
    ((70, 16, 8, 8), (16, 16, 3, 3), (1, 1), (1, 1), (1, 1), 1),     # batch over one 64-wide K block
    ((4, 64, 14, 14), (128, 64, 3, 3), (1, 1), (2, 2), (1, 1), 1),   # stride 2, ResNet-like
    ((3, 32, 9, 11), (32, 8, 3, 3), (1, 1), (1, 1), (1, 1), 4),      # groups
    ((2, 8, 10, 10), (8, 8, 1, 1), (1, 1), (1, 1), (1, 1), 1),       # padding larger than the filter reach
    ((2, 16, 13, 13), (16, 16, 3, 3), (0, 0), (2, 2), (1, 1), 1),    # stride leaves the last input row unused
]


def grad_case(xs, ws, pad, stride, dil, seed=2):
    x, w, b = cases.conv_inputs(xs, ws, with_zeros=True)
    oshape = oracle.conv_out_shape(xs, ws, pad, stride, dil)
    rng = np.random.RandomState(seed)
    dy = rng.randn(*oshape).astype(np.float32)
    g0 = [rng.randn(*xs).astype(np.float32), rng.randn(*ws).astype(np.float32), rng.randn(ws[0]).astype(np.float32)]
    return x, w, b, dy, g0


def check(got, want, exact):
    for name, g, w, e in zip(("dx", "dw", "db"), got, want, exact):
        assert cases.rel_rms(g.cpu().numpy(), w) < TOL, name
        assert cases.rel_rms(g.cpu().numpy(), e) < TOL, name


@pytest.mark.parametrize("xs,ws,pad,stride,dil,grp", BACKWARD_CASES)
@pytest.mark.parametrize("accum", [False, True])
def test_binary_weight_convolution_backward(F, xs, ws, pad, stride, dil, grp, accum):
    x, w, b, dy, g0 = grad_case(xs, ws, pad, stride, dil)
    wb, al = torch.zeros(ws, device="cuda"), torch.zeros(ws[0], device="cuda")
    F.binary_weight_convolution(dev(x), dev(w), wb, al, dev(b), 1, pad, stride, dil, grp, 1.0)
    ac = (accum,) * 3
    got = F.binary_weight_convolution_backward(dev(x), wb, al, dev(dy), 1, pad, stride, dil, grp, accum=ac,
                                               grads=[dev(g) for g in g0])
    F.check_device_status()
    want = oracle.binary_weight_convolution_backward(x, w, dy, pad, stride, dil, grp, 1.0, accum=ac, grads=g0)
    exact = oracle.binary_weight_convolution_backward(x, w, dy, pad, stride, dil, grp, 1.0, accum=ac, grads=g0,
                                                      f64=True)
    check(got, want, exact)


@pytest.mark.parametrize("xs,ws,pad,stride,dil,grp", BACKWARD_CASES[:7])
def test_binary_connect_convolution_backward(F, xs, ws, pad, stride, dil, grp):
    x, w, b, dy, g0 = grad_case(xs, ws, pad, stride, dil)
    wb = torch.zeros(ws, device="cuda")
    F.binary_connect_convolution(dev(x), dev(w), wb, dev(b), 1, pad, stride, dil, grp, 0.0)
    got = F.binary_connect_convolution_backward(dev(x), wb, dev(dy), 1, pad, stride, dil, grp)
    F.check_device_status()
    want = oracle.binary_connect_convolution_backward(x, w, dy, pad, stride, dil, grp, 0.0)
    exact = oracle.binary_connect_convolution_backward(x, w, dy, pad, stride, dil, grp, 0.0, f64=True)
    check(got, want, exact)


def test_fixed_point_activations_use_one_piece(F):
    """x = outputs of FixedPointQuantize(n=8): the weight gradient from one bf16 piece of x is as exact."""
    xs, ws, pad, stride, dil, grp = BACKWARD_CASES[6]
    x, w, b, dy, g0 = grad_case(xs, ws, pad, stride, dil)
    xq = oracle.fixed_point_quantize(x, True, 8, 2.0 ** -4)
    wb, al = torch.zeros(ws, device="cuda"), torch.zeros(ws[0], device="cuda")
    F.binary_weight_convolution(dev(xq), dev(w), wb, al, None, 1, pad, stride, dil, grp, 1.0, fixed_point_delta=2.0 ** -4)
    got = F.binary_weight_convolution_backward(dev(xq), wb, al, dev(dy), 1, pad, stride, dil, grp,
                                               fixed_point_delta=2.0 ** -4)
    F.check_device_status()
    exact = oracle.binary_weight_convolution_backward(xq, w, dy, pad, stride, dil, grp, 1.0, f64=True)
    want = oracle.binary_weight_convolution_backward(xq, w, dy, pad, stride, dil, grp, 1.0)
    check(got, want, exact)


def test_partial_propagation(F):
    xs, ws, pad, stride, dil, grp = BACKWARD_CASES[2]
    x, w, b, dy, g0 = grad_case(xs, ws, pad, stride, dil)
    wb, al = torch.zeros(ws, device="cuda"), torch.zeros(ws[0], device="cuda")
    F.binary_weight_convolution(dev(x), dev(w), wb, al, None, 1, pad, stride, dil, grp, 1.0)
    g = [dev(a) for a in g0]
    out = F.binary_weight_convolution_backward(dev(x), wb, al, dev(dy), 1, pad, stride, dil, grp,
                                               propagate_down=(True, False, False), grads=g)
    assert torch.equal(out[1], dev(g0[1])) and torch.equal(out[2], dev(g0[2]))
    want = oracle.binary_weight_convolution_backward(x, w, dy, pad, stride, dil, grp, 1.0,
                                                     propagate_down=(True, False, False), grads=g0)
    assert cases.rel_rms(out[0].cpu().numpy(), want[0]) < TOL


@pytest.mark.parametrize("xs,ws,pad,stride", [((4, 3, 32, 32), (16, 3, 7, 7), (3, 3), (2, 2)),
                                              ((3, 5, 12, 10), (8, 5, 3, 3), (1, 1), (1, 1))])
@pytest.mark.parametrize("accum", [False, True])
def test_full_precision_convolution_weight_gradient(F, xs, ws, pad, stride, accum):
    x, w, b, dy, g0 = grad_case(xs, ws, pad, stride, (1, 1))
    ac = (False, accum, accum)
    got = F.convolution_backward(dev(x), ws, dev(dy), 1, pad, stride, accum=ac, grads=[None, dev(g0[1]), dev(g0[2])])
    F.check_device_status()
    want = oracle.convolution_backward(x, w, dy, pad, stride, propagate_down=(False, True, True), accum=ac, grads=g0)
    exact = oracle.convolution_backward(x, w, dy, pad, stride, propagate_down=(False, True, True), accum=ac, grads=g0,
                                        f64=True)
    for k in (1, 2):
        assert cases.rel_rms(got[k].cpu().numpy(), want[k]) < TOL
        assert cases.rel_rms(got[k].cpu().numpy(), exact[k]) < TOL
    with pytest.raises(RuntimeError):
        F.convolution_backward(dev(x), ws, dev(dy), 1, pad, stride, propagate_down=(True, True, True))


@pytest.mark.parametrize("xs,ws,pad,stride,dil,grp", BACKWARD_CASES)
@pytest.mark.parametrize("accum", [False, True])
def test_full_precision_convolution_input_gradient(F, xs, ws, pad, stride, dil, grp, accum):
    """dx of the full-precision Convolution (arbitrary fp32 weights, three bf16 pieces each side)."""
    x, w, b, dy, g0 = grad_case(xs, ws, pad, stride, dil)
    pd, ac = (True, False, False), (accum, False, False)
    got = F.convolution_backward(dev(x), ws, dev(dy), 1, pad, stride, dil, grp, propagate_down=pd, accum=ac,
                                 grads=[dev(g0[0]), None, None], weight=dev(w))
    F.check_device_status()
    assert got[1] is None and got[2] is None
    want = oracle.convolution_backward(x, w, dy, pad, stride, dil, grp, propagate_down=pd, accum=ac, grads=g0)
    exact = oracle.convolution_backward(x, w, dy, pad, stride, dil, grp, propagate_down=pd, accum=ac, grads=g0, f64=True)
    assert cases.rel_rms(got[0].cpu().numpy(), want[0]) < TOL
    assert cases.rel_rms(got[0].cpu().numpy(), exact[0]) < TOL
