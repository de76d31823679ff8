"""The sibling-function cases of tests/golden/golden_siblings.npz for any
implementation `impl` with the oracle's numpy signatures (the C restatement on
CPU, the CUDA path on the GPU)."""
import hashlib
import os

import numpy as np

import cases

_G = None


def golden():
    global _G
    if _G is None:
        _G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_siblings.npz"))
    return _G


def same(a, key):
    g = golden()
    a = np.ascontiguousarray(a, np.float32)
    head_ok = np.array_equal(a.ravel()[:64].view(np.uint32), g[key + "_head"].view(np.uint32))
    sha = np.frombuffer(hashlib.sha256(a.tobytes()).digest(), np.uint8)
    return head_ok and np.array_equal(sha, g[key + "_sha"])


def check_binary(impl, name, accum):
    x = cases.binary_act_input()
    dy, dx0 = cases.grad_inputs(x)
    assert same(getattr(impl, name)(x), name + "/y")
    assert same(getattr(impl, name + "_backward")(x, dy, accum, dx0), "%s/dx%d" % (name, accum))


def check_quantize_linear(impl, i):
    shapes, mode, narrow, dtype = cases.QL_GRID[i]
    x, scale, zp = cases.quantize_linear_inputs(*shapes)
    y, zpa = impl.quantize_linear(x, scale, zp, mode, narrow, dtype)
    assert same(zpa, "ql%d/zp" % i)
    assert same(y, "ql%d/y" % i)


def check_linear_rest(impl, i, accum):
    x, scale, zp = cases.quantize_linear_inputs(*cases.QL_SHAPES[i])
    dy, dx0 = cases.grad_inputs(x)
    assert same(impl.dequantize_linear(x, scale, zp), "dql%d/y" % i)
    assert same(impl.quantize_linear_backward(dy, scale, accum, dx0), "ql_bw%d_%d/dx" % (i, accum))
    assert same(impl.dequantize_linear_backward(dy, scale, accum, dx0), "dql_bw%d_%d/dx" % (i, accum))
