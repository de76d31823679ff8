"""Generates tests/golden/golden_siblings.npz: BinarySigmoid / BinaryTanh /
QuantizeLinear / DequantizeLinear outputs and input gradients from the
reference's own CPU functions (oracle/_ref/libnnabla_ref.so).

    python tests/golden/make_golden_siblings.py

Inputs are regenerated from tests/cases.py (seeded); outputs are stored as a
SHA-256 of their bytes plus their first 64 values.
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


def put(g, key, a):
    a = np.ascontiguousarray(a, np.float32)
    g[key + "_sha"] = np.frombuffer(hashlib.sha256(a.tobytes()).digest(), np.uint8)
    g[key + "_head"] = a.ravel()[:64]


def main():
    g = {}
    x = cases.binary_act_input()
    dy, dx0 = cases.grad_inputs(x)
    for name in ("binary_sigmoid", "binary_tanh"):
        put(g, name + "/y", getattr(ref, name)(x))
        for accum in (False, True):
            put(g, "%s/dx%d" % (name, accum), getattr(ref, name + "_backward")(x, dy, accum, dx0))
    for i, (shapes, mode, narrow, dtype) in enumerate(cases.QL_GRID):
        x, scale, zp = cases.quantize_linear_inputs(*shapes)
        y, zpa = ref.quantize_linear(x, scale, zp, mode, narrow, dtype)
        put(g, "ql%d/y" % i, y)
        put(g, "ql%d/zp" % i, zpa)
    for i, shapes in enumerate(cases.QL_SHAPES):
        x, scale, zp = cases.quantize_linear_inputs(*shapes)
        dy, dx0 = cases.grad_inputs(x)
        put(g, "dql%d/y" % i, ref.dequantize_linear(x, scale, zp))
        for accum in (False, True):
            put(g, "ql_bw%d_%d/dx" % (i, accum), ref.quantize_linear_backward(x, scale, zp, dy, accum=accum, dx=dx0))
            put(g, "dql_bw%d_%d/dx" % (i, accum), ref.dequantize_linear_backward(x, scale, zp, dy, accum=accum, dx=dx0))
    out = os.path.join(HERE, "golden_siblings.npz")
    np.savez_compressed(out, **g)
    print("wrote", out, os.path.getsize(out), "bytes,", len(g), "arrays")


if __name__ == "__main__":
    main()
