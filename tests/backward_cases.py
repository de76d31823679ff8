"""The quantizer backward cases of tests/golden/golden_backward.npz, written
once for any implementation `impl` that offers
fixed_point_quantize_backward / pow2_quantize_backward /
min_max_quantize (forward) / min_max_quantize_backward with the oracle's
signatures over numpy arrays: the C restatement on CPU (tests/test_golden.py)
and the CUDA path (tests/test_quantize_backward_gpu.py)."""
import itertools

import numpy as np

import cases
from golden_util import bits, golden_backward, sha

FLAGS = list(itertools.product([True, False], [False, True]))  # ste_fine_grained, accum
POW2_CASES = cases.POW2_GRID + [(True, True, 8, 1)]


def check_fxp(impl, i, fine, accum):
    g = golden_backward()
    sign, n, delta = cases.FXP_GRID[i]
    x = cases.fxp_backward_input(delta, n - 1 if sign else n)
    dy, dx0 = cases.grad_inputs(x)
    got = impl.fixed_point_quantize_backward(x, dy, sign, n, delta, fine, accum, dx0)
    assert np.array_equal(bits(got), bits(g[f"fxp{i}_{int(fine)}{int(accum)}/dx"]))


def check_pow2(impl, i, fine, accum):
    g = golden_backward()
    sign, wz, n, m = POW2_CASES[i]
    x = cases.pow2_backward_input(m)
    dy, dx0 = cases.grad_inputs(x)
    got = impl.pow2_quantize_backward(x, dy, sign, wz, n, m, fine, accum, dx0)
    k = f"pow2_{i}_{int(fine)}{int(accum)}"
    assert np.array_equal(bits(got[:256]), bits(g[k + "/dx_head"]))
    assert np.array_equal(sha(got), g[k + "/dx_sha"])


def check_minmax(impl, i, fine, accum):
    g = golden_backward()
    shapes, decay, xmm, ema = cases.MINMAX_GRID[i]
    x, qmin, qmax, lmin, lmax = cases.minmax_inputs(*shapes)
    dy, dx0 = cases.grad_inputs(x)
    rng = np.random.RandomState(3)
    g0 = [dx0, rng.randn(*qmin.shape).astype(np.float32), rng.randn(*qmin.shape).astype(np.float32)]
    ranges = not (xmm or ema)
    fwd = impl.min_max_quantize(x, qmin, qmax, lmin, lmax, decay, xmm, ema, 0.01)
    fmin, fmax = fwd[1], fwd[2]
    dx, gmin, gmax = impl.min_max_quantize_backward(x, fmin, fmax, lmin, lmax, dy, xmm, ema, fine,
                                                    (True, ranges, ranges), (accum,) * 3, g0)
    k = f"minmax{i}_{int(fine)}{int(accum)}"
    assert np.array_equal(bits(dx.ravel()[:256]), bits(g[k + "/dx_head"]))
    assert np.array_equal(sha(dx), g[k + "/dx_sha"])
    if ranges:
        per_q = x.size // qmin.size
        tol = 1e-6 * per_q ** 0.5 * (np.abs(dy).max() + 1)
        assert np.allclose(gmin, g[k + "/g_qr_min"], rtol=1e-5, atol=tol)
        assert np.allclose(gmax, g[k + "/g_qr_max"], rtol=1e-5, atol=tol)
    else:  # the reference returns before the range gradients: buffers untouched
        assert np.array_equal(bits(gmin), bits(g0[1])) and np.array_equal(bits(gmax), bits(g0[2]))
