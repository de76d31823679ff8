"""Generates tests/golden/golden_backward.npz: input gradients of the three
quantizers as computed by Function::backward of the reference's own CPU
functions (oracle/_ref/libnnabla_ref.so, built by `make -C oracle ref`).

    python tests/golden/make_golden_backward.py

Inputs are regenerated from tests/cases.py (seeded); only the reference's
outputs are stored, the larger ones as a SHA-256 of their bytes plus their
first 256 values. tests/test_golden.py checks the C restatement against
them, tests/test_quantize_backward_gpu.py the CUDA path.
"""
import hashlib
import itertools
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

import cases  # noqa: E402
from oracle import ref  # noqa: E402

FLAGS = list(itertools.product([True, False], [False, True]))  # ste_fine_grained, accum


def sha(a):
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(a, np.float32).tobytes()).digest(), np.uint8)


def main():
    g = {}
    for i, (sign, n, delta) in enumerate(cases.FXP_GRID):
        x = cases.fxp_backward_input(delta, n - 1 if sign else n)
        dy, dx0 = cases.grad_inputs(x)
        for fine, accum in FLAGS:
            g[f"fxp{i}_{int(fine)}{int(accum)}/dx"] = ref.fixed_point_quantize_backward(x, dy, sign, n, delta, fine,
                                                                                        accum, dx0)
    for i, (sign, wz, n, m) in enumerate(cases.POW2_GRID + [(True, True, 8, 1)]):
        x = cases.pow2_backward_input(m)
        dy, dx0 = cases.grad_inputs(x)
        for fine, accum in FLAGS:
            dx = ref.pow2_quantize_backward(x, dy, sign, wz, n, m, fine, accum, dx0)
            g[f"pow2_{i}_{int(fine)}{int(accum)}/dx_sha"] = sha(dx)
            g[f"pow2_{i}_{int(fine)}{int(accum)}/dx_head"] = dx[:256]
    for i, (shapes, decay, xmm, ema) in enumerate(cases.MINMAX_GRID):
        x, qmin, qmax, lmin, lmax = cases.minmax_inputs(*shapes)
        dy, dx0 = cases.grad_inputs(x)
        rng = np.random.RandomState(3)
        g0 = [dx0, rng.randn(*qmin.shape).astype(np.float32), rng.randn(*qmin.shape).astype(np.float32)]
        ranges = not (xmm or ema)
        for fine, accum in FLAGS:
            dx, gmin, gmax = ref.min_max_quantize_backward(x, qmin, qmax, lmin, lmax, dy, decay, xmm, ema, fine, 0.01,
                                                           (True, ranges, ranges), (accum,) * 3, g0)
            k = f"minmax{i}_{int(fine)}{int(accum)}"
            g[k + "/dx_sha"], g[k + "/dx_head"] = sha(dx), dx.ravel()[:256]
            g[k + "/g_qr_min"], g[k + "/g_qr_max"] = gmin, gmax
    out = os.path.join(HERE, "golden_backward.npz")
    np.savez_compressed(out, **g)
    print("wrote", out, os.path.getsize(out), "bytes,", len(g), "arrays")


if __name__ == "__main__":
    main()
