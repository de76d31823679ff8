"""GPU parity of the affine backward passes (Affine, BinaryWeightAffine,
BinaryConnectAffine) through the C ABI against the oracle: every gradient
within 1e-5 of its RMS (the tolerance stated for GEMM outputs), judged
against the float64 product as well."""
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


def grad_case(xs, ws, base_axis, seed=1):
    x, w, b = cases.affine_inputs(xs, ws, with_zeros=True)
    rng = np.random.RandomState(seed)
    dy = rng.randn(*(tuple(xs[:base_axis]) + tuple(ws[1:]))).astype(np.float32)
    g0 = [rng.randn(*xs).astype(np.float32), rng.randn(*ws).astype(np.float32),
          rng.randn(*ws[1:]).astype(np.float32)]
    return x, w, b, dy, g0


def check(got, want, exact):
    for g, w, e in zip(got, want, exact):
        assert cases.rel_rms(g.cpu().numpy(), w) < TOL
        assert cases.rel_rms(g.cpu().numpy(), e) < TOL


SHAPES = cases.AFFINE_CASES + [((130, 200), (200, 72), 1), ((64, 1024), (1024, 512), 1)]


@pytest.mark.parametrize("xs,ws,base_axis", SHAPES)
@pytest.mark.parametrize("accum", [False, True])
def test_binary_weight_affine_backward(F, xs, ws, base_axis, accum):
    x, w, b, dy, g0 = grad_case(xs, ws, base_axis)
    wb, al = torch.zeros(ws, device="cuda"), torch.zeros(int(np.prod(ws[1:])), device="cuda")
    F.binary_weight_affine(dev(x), dev(w), wb, al, dev(b), base_axis, 1.0)
    ac = (accum,) * 3
    got = F.binary_weight_affine_backward(dev(x), wb, al, dev(dy), base_axis, accum=ac, grads=[dev(g) for g in g0])
    F.check_device_status()
    want = oracle.binary_weight_affine_backward(x, w, dy, base_axis, 1.0, accum=ac, grads=g0)
    exact = oracle.binary_weight_affine_backward(x, w, dy, base_axis, 1.0, accum=ac, grads=g0, f64=True)
    check(got, want, exact)


@pytest.mark.parametrize("xs,ws,base_axis", SHAPES)
@pytest.mark.parametrize("qzt", [0.0, -1.0])
def test_binary_connect_affine_backward(F, xs, ws, base_axis, qzt):
    x, w, b, dy, g0 = grad_case(xs, ws, base_axis)
    wb = torch.zeros(ws, device="cuda")
    F.binary_connect_affine(dev(x), dev(w), wb, dev(b), base_axis, qzt)
    got = F.binary_connect_affine_backward(dev(x), wb, dev(dy), base_axis)
    F.check_device_status()
    want = oracle.binary_connect_affine_backward(x, w, dy, base_axis, qzt)
    exact = oracle.binary_connect_affine_backward(x, w, dy, base_axis, qzt, f64=True)
    check(got, want, exact)


@pytest.mark.parametrize("xs,ws,base_axis", SHAPES)
@pytest.mark.parametrize("accum", [False, True])
def test_affine_backward(F, xs, ws, base_axis, accum):
    x, w, b, dy, g0 = grad_case(xs, ws, base_axis)
    ac = (accum,) * 3
    got = F.affine_backward(dev(x), dev(w), dev(dy), base_axis, accum=ac, grads=[dev(g) for g in g0])
    F.check_device_status()
    want = oracle.affine_backward(x, w, dy, base_axis, accum=ac, grads=g0)
    exact = oracle.affine_backward(x, w, dy, base_axis, accum=ac, grads=g0, f64=True)
    check(got, want, exact)


def test_partial_propagation_leaves_buffers_alone(F):
    xs, ws, base_axis = SHAPES[2]
    x, w, b, dy, g0 = grad_case(xs, ws, base_axis)
    g = [dev(a) for a in g0]
    out = F.affine_backward(dev(x), dev(w), dev(dy), base_axis, propagate_down=(False, True, False), grads=g)
    assert out[0] is g[0] and torch.equal(g[0], dev(g0[0])) and torch.equal(g[2], dev(g0[2]))
    want = oracle.affine_backward(x, w, dy, base_axis, propagate_down=(False, True, False), grads=g0)
    assert cases.rel_rms(out[1].cpu().numpy(), want[1]) < TOL


def test_backward_shape_errors(F):
    x, w = torch.zeros(4, 8, device="cuda"), torch.zeros(8, 6, device="cuda")
    with pytest.raises(RuntimeError):
        F.affine_backward(x, w, torch.zeros(4, 5, device="cuda"))
    with pytest.raises(RuntimeError):
        F.affine_backward(x, w, torch.zeros(4, 6, device="cuda"), accum=(True, False, False))
