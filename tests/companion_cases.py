"""Seeded inputs of the training-side companion cases stored in tests/golden/golden_companions.npz
(made by tests/golden/make_golden_companions.py from the reference build). Shared by the generator,
the CPU check of the C restatement (tests/test_golden.py) and the GPU tests."""
import numpy as np

BN_SHAPES = [(4, 3, 5, 7), (3, 16, 8, 8), (16, 4, 3, 3)]
POOL_CASES = [((2, 3, 9, 11), (3, 3), (2, 2), (1, 1), True), ((2, 2, 7, 10), (3, 2), (1, 2), (1, 0), False),
              ((2, 4, 12, 12), (3, 3), (1, 1), (1, 1), True)]


def bn_case(i):
    shape = BN_SHAPES[i]
    rng = np.random.RandomState(100 + i)
    C = shape[1]
    p = (1, C, 1, 1)
    x = (rng.randn(*shape) * 2 + 0.5).astype(np.float32)
    dy = rng.randn(*shape).astype(np.float32)
    beta, gamma = rng.randn(*p).astype(np.float32), (rng.rand(*p) + 0.5).astype(np.float32)
    mean, var = (0.1 * rng.randn(*p)).astype(np.float32), (rng.rand(*p) + 0.5).astype(np.float32)
    dmean, dvar = rng.randn(*p).astype(np.float32), rng.randn(*p).astype(np.float32)
    g0 = [rng.randn(*shape).astype(np.float32), rng.randn(*p).astype(np.float32), rng.randn(*p).astype(np.float32)]
    return dict(x=x, dy=dy, beta=beta, gamma=gamma, mean=mean, var=var, dmean=dmean, dvar=dvar, g0=g0)


def pool_case(i):
    shape, kernel, stride, pad, ib = POOL_CASES[i]
    rng = np.random.RandomState(200 + i)
    x = rng.randint(-2, 3, size=shape).astype(np.float32)  # many ties: the first maximum must win
    x[rng.rand(*shape) < 0.2] = -0.0
    return dict(x=x, kernel=kernel, stride=stride, pad=pad, ib=ib, rng=rng,
                g0=rng.randn(*shape).astype(np.float32))


def elementwise_case():
    rng = np.random.RandomState(300)
    shape = (3, 4, 5, 6)
    x = rng.randn(*shape).astype(np.float32)
    x[rng.rand(*shape) < 0.2] = 0.0
    return dict(x=x, dy=rng.randn(*shape).astype(np.float32), g0=rng.randn(*shape).astype(np.float32),
                dyp=rng.randn(3, 4, 1, 1).astype(np.float32))
