"""Generates tests/golden/golden.npz from the reference's own CPU functions.

Run where the reference checkout is present and `make -C oracle ref` has built
oracle/_ref/libnnabla_ref.so:

    python tests/golden/make_golden.py

Every array stored under "<case>/out*" was produced by the reference's
compiled C++ ("cpu:float" context) on the inputs stored (or regenerated from
the seed) beside it; tests/test_golden.py checks the C restatement and the
GPU parity tests check the CUDA path against them. For the large BASELINE
configurations only a SHA-256 of the reference output bytes is stored.
"""
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

import cases  # noqa: E402
from oracle import ref  # noqa: E402


def sha(a):
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(a, np.float32).tobytes()).digest(), np.uint8)


def main():
    g = {}
    for i, (sign, n, delta) in enumerate(cases.FXP_GRID):
        n_eff = n - 1 if sign else n
        x = np.concatenate([cases.fxp_input((2, 3, 50)).ravel(), cases.edge_values_fxp(np.float32(delta), n_eff)])
        g[f"fxp{i}/x"] = x
        g[f"fxp{i}/args"] = np.array([sign, n, delta], np.float64)
        g[f"fxp{i}/out"] = ref.fixed_point_quantize(x, sign, n, delta)
    xp = np.concatenate([cases.fxp_input((2, 3, 50)).ravel(), cases.edge_values_pow2()])
    g["pow2/x"] = xp
    for i, (sign, wz, n, m) in enumerate(cases.POW2_GRID + [(True, True, 8, 1)]):
        g[f"pow2_{i}/args"] = np.array([sign, wz, n, m], np.float64)
        g[f"pow2_{i}/out"] = ref.pow2_quantize(xp, sign, wz, n, m)
    for i, (shapes, decay, xmm, ema) in enumerate(cases.MINMAX_GRID):
        x, qmin, qmax, lmin, lmax = cases.minmax_inputs(*shapes)
        y, amin, amax = ref.min_max_quantize(x, qmin, qmax, lmin, lmax, decay, xmm, ema, True, 0.01)
        g[f"minmax{i}/args"] = np.array([decay, xmm, ema, 0.01], np.float64)
        g[f"minmax{i}/xshape"] = np.array(shapes[0])
        g[f"minmax{i}/qshape"] = np.array(shapes[1])
        g[f"minmax{i}/out_sha"] = sha(y)
        g[f"minmax{i}/out_head"] = y.ravel()[:256]
        g[f"minmax{i}/out_qr_min"] = amin
        g[f"minmax{i}/out_qr_max"] = amax
    for i, (xs, ws, ba) in enumerate(cases.AFFINE_CASES):
        for qzt in cases.QZT:
            x, w, b = cases.affine_inputs(xs, ws, with_zeros=True)
            y, wb, al = ref.binary_weight_affine(x, w, b, ba, qzt)
            k = f"bwa{i}_{int(qzt)}"
            g[k + "/out_y"], g[k + "/out_wb"], g[k + "/out_alpha"] = y, wb, al
            y, wb = ref.binary_connect_affine(x, w, b, ba, qzt)
            k = f"bca{i}_{int(qzt)}"
            g[k + "/out_y"], g[k + "/out_wb"] = y, wb
    for i, (xs, ws, pad, stride, dil, grp) in enumerate(cases.CONV_CASES):
        x, w, b = cases.conv_inputs(xs, ws, with_zeros=True)
        y, wb, al = ref.binary_weight_convolution(x, w, b, 1, pad, stride, dil, grp, 1.0)
        g[f"bwc{i}/out_y"], g[f"bwc{i}/out_wb"], g[f"bwc{i}/out_alpha"] = y, wb, al
        y, wb = ref.binary_connect_convolution(x, w, b, 1, pad, stride, dil, grp, 1.0)
        g[f"bcc{i}/out_y"], g[f"bcc{i}/out_wb"] = y, wb
    # BASELINE configurations at sizes the CPU finishes in seconds: digests only.
    rng = np.random.RandomState(0)
    x = rng.uniform(-4, 4, 1 << 20).astype(np.float32)
    one = lambda v: np.array([v], np.float32)
    g["cfg2_fxp/sha"] = sha(ref.fixed_point_quantize(x, True, 8, 2.0 ** -4))
    g["cfg2_pow2/sha"] = sha(ref.pow2_quantize(x, True, True, 8, 1))
    g["cfg2_minmax/sha"] = sha(ref.min_max_quantize(x, one(-4), one(4), one(0), one(255))[0])
    rng = np.random.RandomState(0)
    x = rng.randn(256, 1024).astype(np.float32)
    w = (0.02 * rng.randn(1024, 4096)).astype(np.float32)
    y, wb, al = ref.binary_weight_affine(x, w, np.zeros(4096, np.float32), 1, 1.0)
    g["cfg1/wb_sha"] = sha(wb)
    g["cfg1/alpha"] = al
    g["cfg1/y_rows"] = y[:4]           # first four output rows
    g["cfg1/y_rms"] = np.array([np.sqrt(np.mean(y.astype(np.float64) ** 2))])
    np.savez_compressed(os.path.join(HERE, "golden.npz"), **g)
    print("wrote golden.npz:", os.path.getsize(os.path.join(HERE, "golden.npz")), "bytes,", len(g), "arrays")


if __name__ == "__main__":
    main()
