"""The C restatement of the training-side companions (batch-statistics BatchNormalization and
the backward passes of BatchNormalization, ReLU, Add2, MaxPooling, GlobalAveragePooling)
against the reference's own compiled code. Elementwise results bit for bit; the statistics
and parameter gradients are sequential fp32 sums in both, so they are bit-identical too."""
import numpy as np
import pytest

from oracle import oracle, ref

pytestmark = pytest.mark.skipif(not ref.available(), reason="oracle/_ref (reference build) not present")


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def stats(C, rng):
    shape = (1, C, 1, 1)
    return [a.astype(np.float32).reshape(shape) for a in
            (rng.randn(C), rng.rand(C) + 0.5, 0.1 * rng.randn(C), rng.rand(C) + 0.5)]  # beta, gamma, mean, var


@pytest.mark.parametrize("shape", [(4, 3, 5, 7), (2, 8, 1, 1), (3, 5, 6, 6), (16, 4, 3, 3)])
def test_batch_statistics_forward(shape):
    rng = np.random.RandomState(sum(shape))
    x = (rng.randn(*shape) * 2 + 0.5).astype(np.float32)
    beta, gamma, mean, var = stats(shape[1], rng)
    want = ref.batch_normalization_batch(x, beta, gamma, mean, var, decay_rate=0.9, eps=1e-5)
    got = oracle.batch_norm_batch(x, beta, gamma, mean, var, eps=1e-5, decay_rate=0.9)
    for w, g in zip(want, got):
        assert np.array_equal(bits(w).reshape(-1), bits(g).reshape(-1))


@pytest.mark.parametrize("shape", [(4, 3, 5, 7), (3, 5, 6, 6)])
@pytest.mark.parametrize("accum", [(False, False, False), (True, True, True)])
@pytest.mark.parametrize("batch_stat", [True, False])
def test_batch_normalization_backward(shape, accum, batch_stat):
    rng = np.random.RandomState(sum(shape) + int(batch_stat))
    x = (rng.randn(*shape) * 2 + 0.5).astype(np.float32)
    dy = rng.randn(*shape).astype(np.float32)
    beta, gamma, mean, var = stats(shape[1], rng)
    g0 = [rng.randn(*shape).astype(np.float32), rng.randn(*beta.shape).astype(np.float32),
          rng.randn(*beta.shape).astype(np.float32)]
    dmean = rng.randn(*mean.shape).astype(np.float32) if batch_stat else None
    dvar = rng.randn(*mean.shape).astype(np.float32) if batch_stat else None
    want = ref.batch_normalization_backward(x, beta, gamma, mean, var, dy, batch_stat=batch_stat, dmean=dmean,
                                            dvar=dvar, accum=accum, grads=g0)
    if batch_stat:
        _, m, v, _, _ = oracle.batch_norm_batch(x, beta, gamma, mean, var)
    else:
        m, v = mean, var
    got = oracle.batch_norm_backward(x, dy, gamma, m, v, batch_stat=batch_stat, dmean=dmean, dvar=dvar, accum=accum,
                                     grads=g0)
    for w, g in zip(want, got):
        assert np.array_equal(bits(w).reshape(-1), bits(g).reshape(-1))


@pytest.mark.parametrize("accum", [False, True])
def test_relu_add2_gap_backward(accum):
    rng = np.random.RandomState(3)
    x = rng.randn(3, 4, 5, 6).astype(np.float32)
    x[rng.rand(*x.shape) < 0.2] = 0.0
    dy = rng.randn(*x.shape).astype(np.float32)
    g0 = rng.randn(*x.shape).astype(np.float32)
    assert np.array_equal(bits(ref.relu_backward(x, dy, accum, g0)),
                          bits(oracle.relu_backward(oracle.relu(x), dy, accum, g0)))
    ga, gb = ref.add2_backward(x, x[::-1].copy(), dy, (accum, accum), (g0, g0))
    assert np.array_equal(bits(ga), bits(oracle.add2_backward(dy, accum, g0)))
    assert np.array_equal(bits(gb), bits(oracle.add2_backward(dy, accum, g0)))
    dyp = rng.randn(3, 4, 1, 1).astype(np.float32)
    assert np.array_equal(bits(ref.global_average_pooling_backward(x, dyp, accum, g0)),
                          bits(oracle.global_average_pooling_backward(x.shape, dyp, accum, g0)))


@pytest.mark.parametrize("shape,kernel,stride,pad,ib", [((2, 3, 9, 11), (3, 3), (2, 2), (1, 1), True),
                                                        ((1, 2, 8, 8), (2, 2), (2, 2), (0, 0), True),
                                                        ((2, 2, 7, 10), (3, 2), (1, 2), (1, 0), False),
                                                        ((1, 1, 12, 12), (3, 3), (1, 1), (1, 1), True)])
@pytest.mark.parametrize("accum", [False, True])
def test_max_pooling_backward(shape, kernel, stride, pad, ib, accum):
    rng = np.random.RandomState(sum(shape))
    x = rng.randint(-2, 3, size=shape).astype(np.float32)  # many ties: the first maximum must win
    x[rng.rand(*shape) < 0.2] = -0.0
    y = oracle.max_pooling(x, kernel, stride, ib, pad)
    dy = rng.randn(*y.shape).astype(np.float32)
    g0 = rng.randn(*shape).astype(np.float32)
    want = ref.max_pooling_backward(x, dy, kernel, stride, ib, pad, accum, g0)
    got = oracle.max_pooling_backward(x, dy, kernel, stride, ib, pad, accum, g0)
    assert np.array_equal(bits(want), bits(got))
