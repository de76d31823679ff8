"""Seeded INQAffine cases shared by the CPU and GPU tests."""
import numpy as np

# (x shape, weight shape, num_bits, inq_iterations, forward passes)
CASES = [((4, 6), (6, 5), 4, [5], 1), ((4, 6), (6, 5), 4, [0, 9], 1), ((4, 6), (6, 5), 4, [0], 1),
         ((8, 64), (64, 33), 3, [0, 1, 2], 3), ((8, 64), (64, 33), 5, [1, 3], 4), ((3, 128), (128, 40), 4, [0, 2], 2),
         ((2, 3, 16), (48, 7), 2, [0, 1], 2), ((5, 32), (32, 32), 8, [2], 3)]


# (x shape NCHW, weight shape, pad, stride, dilation, group, num_bits, inq_iterations, forward passes)
CONV_CASES = [((2, 3, 9, 9), (8, 3, 3, 3), (1, 1), (1, 1), (1, 1), 1, 4, [0, 2], 3),
              ((2, 8, 12, 10), (16, 8, 3, 3), (1, 0), (2, 1), (1, 1), 1, 3, [1, 2], 3),
              ((1, 16, 14, 14), (32, 16, 1, 1), (0, 0), (1, 1), (1, 1), 1, 5, [0], 1),
              ((3, 4, 8, 8), (6, 4, 3, 3), (2, 2), (1, 1), (2, 2), 1, 2, [0, 1, 3], 4)]


def _weights(rng, ws):
    # magnitudes over many binades, some of them just around 1.5 * 2^e (where the exponent rule steps), no two
    # equal (the order among equal magnitudes is unspecified in the reference)
    w = (rng.randn(*ws) * np.exp(rng.uniform(-4, 4, size=ws))).astype(np.float32)
    flat = w.ravel()
    near = flat[::7]
    k = np.arange(near.size, dtype=np.float32) - near.size // 2
    flat[::7] = (np.sign(near) * np.float32(1.5) * np.exp2(np.floor(np.log2(np.abs(near)))) *
                 (1 + k * np.float32(2.0 ** -22))).astype(np.float32)
    while np.unique(np.abs(flat)).size != flat.size:
        _, first = np.unique(np.abs(flat), return_index=True)
        dup = np.setdiff1d(np.arange(flat.size), first)
        flat[dup] *= np.float32(1 + 2.0 ** -18)
    return w


def inputs(i):
    xs, ws, bits, its, passes = CASES[i]
    rng = np.random.RandomState(40 + i)
    x = rng.randn(*xs).astype(np.float32)
    w = _weights(rng, ws)
    ind = np.zeros(ws, np.float32)
    b = rng.randn(ws[1]).astype(np.float32)
    return x, w, ind, b, bits, its, passes


def conv_inputs(i):
    xs, ws, pad, stride, dilation, group, bits, its, passes = CONV_CASES[i]
    rng = np.random.RandomState(140 + i)
    x = rng.randn(*xs).astype(np.float32)
    w = _weights(rng, ws)
    ind = np.zeros(ws, np.float32)
    b = rng.randn(ws[0]).astype(np.float32)
    return x, w, ind, b, pad, stride, dilation, group, bits, its, passes
