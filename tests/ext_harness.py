"""ctypes driver of ext/_build/libnnabla_b200_runner.so (ext/runner, linked against the extension
ext/_build/libnnabla_ext_b200.so and the host library): runs a function created
through nnabla's registry on either the reference's "cpu:float" context or the
extension's "b200:float" context."""
import ctypes
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(ROOT, "ext", "_build", "libnnabla_b200_runner.so")
_lib = None


class _Tensor(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("ndim", ctypes.c_int32), ("shape", ctypes.c_int64 * 8)]


def available():
    return os.path.exists(LIB_PATH)


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.nbext_last_error.restype = ctypes.c_char_p
    return _lib


def init():
    if lib().nbext_init() != 0:
        raise RuntimeError(lib().nbext_last_error().decode())


def forward(backend, op, scalars, ivecs, inputs, n_out=1, prequant=None, repeat=1):
    """Returns (outputs, inputs_after, function_name); `repeat` forward passes of the one function instance."""
    L = lib()
    ins = [np.ascontiguousarray(a, dtype=np.float32).copy() for a in inputs if a is not None]
    s = (ctypes.c_double * max(1, len(scalars)))(*[float(v) for v in scalars])
    flat = [int(v) for vec in ivecs for v in vec]
    iv = (ctypes.c_int32 * max(1, len(flat)))(*flat)
    ivl = (ctypes.c_int32 * max(1, len(ivecs)))(*[len(v) for v in ivecs])
    tin = (_Tensor * len(ins))()
    for t, a in zip(tin, ins):
        t.data, t.ndim = a.ctypes.data, a.ndim
        for d, n in enumerate(a.shape):
            t.shape[d] = n
    pq = None
    if prequant is not None:
        pq = (ctypes.c_float * len(ins))(*[float(v) for v in prequant])
    tout = (_Tensor * n_out)()
    name = ctypes.create_string_buffer(64)

    def call(mode):
        rc = L.nbext_forward(backend.encode(), op.encode(), s, len(scalars), iv, ivl, len(ivecs), tin, len(ins), pq,
                             tout, n_out, mode, name, 64)
        if rc != 0:
            raise RuntimeError(L.nbext_last_error().decode())

    call(0)
    outs = []
    for t in tout:
        a = np.empty(tuple(t.shape[d] for d in range(t.ndim)), dtype=np.float32)
        t.data = a.ctypes.data
        outs.append(a)
    call(int(repeat))
    return outs, ins, name.value.decode()


def backward(backend, op, scalars, ivecs, inputs, out_grads, propagate_down, accum, in_grads):
    """Setup + forward + Function::backward on `backend`. Returns (in_grads_after, outputs, inputs_after)."""
    L = lib()
    ins = [np.ascontiguousarray(a, dtype=np.float32).copy() for a in inputs]
    grads = [np.ascontiguousarray(g, dtype=np.float32).copy().reshape(a.shape) for a, g in zip(ins, in_grads)]
    ogs = [np.ascontiguousarray(g, dtype=np.float32).copy() for g in out_grads]
    outs = [np.empty(g.shape, dtype=np.float32) for g in ogs]
    s = (ctypes.c_double * max(1, len(scalars)))(*[float(v) for v in scalars])
    flat = [int(v) for vec in ivecs for v in vec]
    iv = (ctypes.c_int32 * max(1, len(flat)))(*flat)
    ivl = (ctypes.c_int32 * max(1, len(ivecs)))(*[len(v) for v in ivecs])

    def tensors(arrays):
        t = (_Tensor * len(arrays))()
        for e, a in zip(t, arrays):
            e.data, e.ndim = a.ctypes.data, a.ndim
            for d, n in enumerate(a.shape):
                e.shape[d] = n
        return t
    pd = (ctypes.c_int32 * len(ins))(*[int(bool(v)) for v in propagate_down])
    ac = (ctypes.c_int32 * len(ins))(*[int(bool(v)) for v in accum])
    rc = L.nbext_backward(backend.encode(), op.encode(), s, len(scalars), iv, ivl, len(ivecs), tensors(ins),
                          tensors(grads), len(ins), tensors(outs), tensors(ogs), len(outs), pd, ac)
    if rc != 0:
        raise RuntimeError(L.nbext_last_error().decode())
    return grads, outs, ins
