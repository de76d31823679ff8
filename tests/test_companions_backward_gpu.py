"""GPU parity of the training side of the companion functions: batch-statistics
BatchNormalization, and the backward passes of BatchNormalization, ReLU, Add2, MaxPooling and
GlobalAveragePooling, against the oracle (itself bit-exact against the reference's CPU code,
tests/test_oracle_companions_backward_vs_reference.py).

Elementwise passes: bit for bit. Per-channel sums (batch statistics, parameter gradients):
the oracle adds sequentially in fp32 as the reference does, the GPU adds block partials, so they
are compared within fp32 summation error, and the elementwise part is then checked bit for bit
with the GPU's own statistics fed to the oracle."""
import numpy as np
import pytest
import torch

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


def params(C, rng):
    return [a.astype(np.float32) for a in (rng.randn(C), rng.rand(C) + 0.5, 0.1 * rng.randn(C), rng.rand(C) + 0.5)]


SHAPES = [(4, 3, 5, 7), (2, 8, 1, 1), (3, 16, 8, 8), (16, 4, 3, 3), (8, 64, 14, 14), (5, 6, 9)]


@pytest.mark.parametrize("shape", SHAPES)
def test_batch_statistics_forward(F, shape):
    rng = np.random.RandomState(sum(shape))
    x = (rng.randn(*shape) * 2 + 0.5).astype(np.float32)
    C = shape[1]
    beta, gamma, rmean, rvar = params(C, rng)
    d_rm, d_rv = dev(rmean), dev(rvar)
    y, m, v = F.batch_normalization(dev(x), dev(beta), dev(gamma), d_rm, d_rv, [1], 0.9, 1e-5, True, True)
    F.check_device_status()
    x3 = x.reshape(shape[0], C, -1)
    wy, wm, wv, wrm, wrv = oracle.batch_norm_batch(x3, beta, gamma, rmean, rvar, 1e-5, 0.9)
    # the statistics against the exact (float64) ones and against the oracle's sequential fp32 sums
    xm = x3.astype(np.float64).mean(axis=(0, 2))
    xv = (x3.astype(np.float64) ** 2).mean(axis=(0, 2)) - xm ** 2
    assert np.allclose(host(m), xm, rtol=1e-6, atol=1e-6) and np.allclose(host(v), xv, rtol=2e-6, atol=2e-6)
    assert np.allclose(host(m), wm, rtol=1e-5, atol=1e-5) and np.allclose(host(v), wv, rtol=1e-4, atol=1e-5)
    assert np.allclose(host(d_rm), wrm, rtol=1e-5, atol=1e-6) and np.allclose(host(d_rv), wrv, rtol=1e-4, atol=1e-5)
    # given the GPU's statistics: the running update and the normalisation bit for bit
    n = x3.shape[0] * x3.shape[2]
    keep = np.float32(1) - np.float32(0.9)
    gm, gv = host(m), host(v)
    assert np.array_equal(bits(host(d_rm)), bits(np.float32(0.9) * rmean + keep * gm))
    if n > 1:
        assert np.array_equal(bits(host(d_rv)),
                              bits(np.float32(0.9) * rvar + keep * gv * np.float32(n) / np.float32(n - 1)))
    assert np.array_equal(bits(host(y)).reshape(-1), bits(oracle.batch_norm_inference(x3, beta, gamma, gm, gv, 1e-5)).reshape(-1))
    assert np.allclose(host(y).reshape(wy.shape), wy, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("accum", [(False, False, False), (True, True, True)])
@pytest.mark.parametrize("batch_stat", [True, False])
def test_batch_normalization_backward(F, shape, accum, batch_stat):
    rng = np.random.RandomState(sum(shape) + int(batch_stat))
    x = (rng.randn(*shape) * 2 + 0.5).astype(np.float32)
    dy = rng.randn(*shape).astype(np.float32)
    C = shape[1]
    beta, gamma, rmean, rvar = params(C, rng)
    x3, dy3 = x.reshape(shape[0], C, -1), dy.reshape(shape[0], C, -1)
    if batch_stat:
        _, m, v, _, _ = oracle.batch_norm_batch(x3, beta, gamma, rmean, rvar)
        dm, dv = rng.randn(C).astype(np.float32), rng.randn(C).astype(np.float32)
    else:
        m, v, dm, dv = rmean, rvar, None, None
    g0 = [rng.randn(*shape).astype(np.float32), rng.randn(C).astype(np.float32), rng.randn(C).astype(np.float32)]
    want = oracle.batch_norm_backward(x3, dy3, gamma, m, v, 1e-5, batch_stat, dm, dv, accum=accum,
                                      grads=[g0[0].reshape(x3.shape), g0[1], g0[2]])
    got = F.batch_normalization_backward(dev(x), dev(dy), dev(gamma), dev(m), dev(v), [1], 1e-5, batch_stat,
                                         None if dm is None else dev(dm), None if dv is None else dev(dv),
                                         accum=accum, grads=[dev(g) for g in g0])
    F.check_device_status()
    scale = np.abs(want[0]).max() + 1e-6
    assert np.abs(host(got[0]).reshape(x3.shape) - want[0]).max() <= 2e-5 * scale
    n = x3.shape[0] * x3.shape[2]
    for k in (1, 2):
        assert np.allclose(host(got[k]), want[k], rtol=2e-5, atol=2e-5 * np.sqrt(n))
    if not batch_stat:  # no sums behind dx: bit for bit
        assert np.array_equal(bits(host(got[0])).reshape(-1), bits(want[0]).reshape(-1))
    # only some gradients asked for
    only = F.batch_normalization_backward(dev(x), dev(dy), dev(gamma), dev(m), dev(v), [1], 1e-5, batch_stat,
                                          None if dm is None else dev(dm), None if dv is None else dev(dv),
                                          propagate_down=(True, False, False), accum=(accum[0], False, False),
                                          grads=[dev(g0[0]), None, None])
    assert only[1] is None and only[2] is None
    assert np.array_equal(bits(host(only[0])), bits(host(got[0])))


@pytest.mark.parametrize("shape", [(3, 4, 5, 6), (2, 3, 7, 7), (1, 1, 1, 5), (2, 16, 32, 32)])
@pytest.mark.parametrize("accum", [False, True])
def test_relu_add2_gap_backward(F, shape, accum):
    rng = np.random.RandomState(sum(shape))
    x = rng.randn(*shape).astype(np.float32)
    x[rng.rand(*shape) < 0.2] = 0.0
    y = oracle.relu(x)
    dy = rng.randn(*shape).astype(np.float32)
    g0 = rng.randn(*shape).astype(np.float32)
    g0[rng.rand(*shape) < 0.1] = -0.0
    init = lambda: dev(g0) if accum else None
    assert np.array_equal(bits(host(F.relu_backward(dev(y), dev(dy), accum, init()))),
                          bits(oracle.relu_backward(y, dy, accum, g0)))
    assert np.array_equal(bits(host(F.add2_backward(dev(dy), accum, init()))), bits(oracle.add2_backward(dy, accum, g0)))
    dyp = rng.randn(shape[0], shape[1], 1, 1).astype(np.float32)
    assert np.array_equal(bits(host(F.global_average_pooling_backward(shape, dev(dyp), accum, init()))),
                          bits(oracle.global_average_pooling_backward(shape, dyp, accum, g0)))


@pytest.mark.parametrize("shape,kernel,stride,pad,ib", [((2, 3, 9, 11), (3, 3), (2, 2), (1, 1), True),
                                                        ((1, 2, 8, 8), (2, 2), (2, 2), (0, 0), True),
                                                        ((2, 2, 7, 10), (3, 2), (1, 2), (1, 0), False),
                                                        ((1, 1, 12, 12), (3, 3), (1, 1), (1, 1), True),
                                                        ((2, 4, 13, 10), (3, 3), (2, 2), (0, 0), False),
                                                        ((2, 8, 56, 56), (3, 3), (2, 2), (1, 1), True)])
@pytest.mark.parametrize("accum", [False, True])
def test_max_pooling_backward(F, shape, kernel, stride, pad, ib, accum):
    rng = np.random.RandomState(sum(shape))
    x = rng.randint(-2, 3, size=shape).astype(np.float32)  # many ties: the first maximum must win
    x[rng.rand(*shape) < 0.2] = -0.0
    yshape = oracle.max_pooling(x, kernel, stride, ib, pad).shape
    dy = rng.randn(*yshape).astype(np.float32)
    g0 = rng.randn(*shape).astype(np.float32)
    got = F.max_pooling_backward(dev(x), dev(dy), kernel, stride, ib, pad, accum, dev(g0) if accum else None)
    assert np.array_equal(bits(host(got)), bits(oracle.max_pooling_backward(x, dy, kernel, stride, ib, pad, accum, g0)))
    # continuous data as well
    x = rng.randn(*shape).astype(np.float32)
    got = F.max_pooling_backward(dev(x), dev(dy), kernel, stride, ib, pad, accum, dev(g0) if accum else None)
    assert np.array_equal(bits(host(got)), bits(oracle.max_pooling_backward(x, dy, kernel, stride, ib, pad, accum, g0)))


def test_against_the_golden_fixtures(F):
    """The committed outputs of the reference build (tests/golden/golden_companions.npz): exact passes
    bit for bit, the passes with per-channel sums within fp32 summation error."""
    import os
    import companion_cases as cc
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_companions.npz"))
    for i in range(len(cc.POOL_CASES)):
        c = cc.pool_case(i)
        for accum in (False, True):
            got = F.max_pooling_backward(dev(c["x"]), dev(g["pool%d/dy" % i]), c["kernel"], c["stride"], c["ib"],
                                         c["pad"], accum, dev(c["g0"]) if accum else None)
            assert np.array_equal(bits(host(got)), bits(g["pool%d/dx_%d" % (i, int(accum))]))
    e = cc.elementwise_case()
    for accum in (False, True):
        init = lambda: dev(e["g0"]) if accum else None
        y = F.relu(dev(e["x"]))
        assert np.array_equal(bits(host(F.relu_backward(y, dev(e["dy"]), accum, init()))), bits(g["relu/dx_%d" % accum]))
        assert np.array_equal(bits(host(F.add2_backward(dev(e["dy"]), accum, init()))), bits(g["add2/dx_%d" % accum]))
        assert np.array_equal(bits(host(F.global_average_pooling_backward(e["x"].shape, dev(e["dyp"]), accum, init()))),
                              bits(g["gap/dx_%d" % accum]))
    for i in range(len(cc.BN_SHAPES)):
        c = cc.bn_case(i)
        rm, rv = dev(c["mean"]), dev(c["var"])
        y, m, v = F.batch_normalization(dev(c["x"]), dev(c["beta"]), dev(c["gamma"]), rm, rv, [1], 0.9, 1e-5, True, True)
        for t, k, tol in ((y, "y", 1e-4), (m, "m", 1e-5), (v, "v", 1e-4), (rm, "rm", 1e-5), (rv, "rv", 1e-4)):
            assert np.allclose(host(t).reshape(-1), g["bn%d/fwd_%s" % (i, k)].reshape(-1), rtol=tol, atol=tol), (i, k)
        n = c["x"].size // c["x"].shape[1]
        for batch_stat in (True, False):
            mm, vv = (g["bn%d/fwd_m" % i], g["bn%d/fwd_v" % i]) if batch_stat else (c["mean"], c["var"])
            for accum in (False, True):
                got = F.batch_normalization_backward(
                    dev(c["x"]), dev(c["dy"]), dev(c["gamma"]), dev(mm), dev(vv), [1], 1e-5, batch_stat,
                    dev(c["dmean"]) if batch_stat else None, dev(c["dvar"]) if batch_stat else None,
                    accum=(accum,) * 3, grads=[dev(a) for a in c["g0"]])
                k = "bn%d/bwd_%d%d" % (i, int(batch_stat), int(accum))
                want = g[k + "_dx"]
                assert np.abs(host(got[0]) - want).max() <= 2e-5 * (np.abs(want).max() + 1e-6)
                assert np.allclose(host(got[1]).reshape(-1), g[k + "_dbeta"].reshape(-1), rtol=2e-5, atol=2e-5 * np.sqrt(n))
                assert np.allclose(host(got[2]).reshape(-1), g[k + "_dgamma"].reshape(-1), rtol=2e-5, atol=2e-5 * np.sqrt(n))
