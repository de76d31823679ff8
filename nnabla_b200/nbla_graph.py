"""nnabla graphs through the runner binding (ext/_build/libnnabla_b200_runner.so).

`Graph(backend)` builds a graph of nnabla's own CgVariable / CgFunction objects
under one context, "cpu:float" (the reference's functions) or "b200:float" (this
repository's extension), and runs it with nnabla's graph engine
(CgVariable::forward, clear_buffer included). Its methods carry the names and
argument order of nnabla.functions for the functions of the quantized-layer
path, so a network written against that namespace (resnet18.Runner) builds the
graph by being called once with graph variables; the backend is the only thing
that differs between the two builds.

It stands in for `import nnabla` + `nnabla_ext.b200`: the nnabla Python package
cannot be built without nnabla's code generator, the C++ core and the extension
can (ext/Makefile).
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "ext", "_build", "libnnabla_b200_runner.so")
_lib = None


def available():
    return os.path.exists(LIB_PATH)


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.nbg_last_error.restype = ctypes.c_char_p
        _lib.nbg_create.restype = ctypes.c_void_p
        _lib.nbg_counter.restype = ctypes.c_longlong
    return _lib


def counter(name):
    """A path counter of the extension ("int8_convolutions", "weight_cache_hits", ...)."""
    return int(lib().nbg_counter(name.encode()))


def reset_counters():
    lib().nbg_reset_counters()


def clear_memory_cache():
    """Returns the unused blocks of the extension's caching allocator to the device
    (what nnabla_ext.b200.clear_memory_cache() calls)."""
    if lib().nnabla_ext_b200_clear_memory_cache() != 0:
        lib().nnabla_ext_b200_last_error.restype = ctypes.c_char_p
        raise RuntimeError(lib().nnabla_ext_b200_last_error().decode())


def _host(a):
    if hasattr(a, "detach"):
        a = a.detach().cpu().numpy()
    return np.ascontiguousarray(a, dtype=np.float32)


class Var:
    """A variable of a Graph (leaf or function output)."""

    def __init__(self, graph, vid):
        self.graph, self.id = graph, vid

    @property
    def shape(self):
        return self.graph.shape(self)


class Graph:
    def __init__(self, backend="b200:float", device_id="0", need_grad=False):
        """need_grad: parameter leaves (arrays passed to the function methods) are created with
        need_grad, so that backward() reaches them."""
        self.backend = backend
        self.need_grad = need_grad
        self._h = ctypes.c_void_p(lib().nbg_create(backend.encode(), str(device_id).encode()))
        if not self._h:
            raise RuntimeError(lib().nbg_last_error().decode())
        self._leaves = {}  # id(array) -> Var, so that a parameter passed twice is one variable
        self._keep = []

    def close(self):
        if self._h:
            lib().nbg_destroy(self._h)
            self._h = None

    def _check(self, rc):
        if rc != 0:
            raise RuntimeError(lib().nbg_last_error().decode())

    # ---- variables -------------------------------------------------------------------
    def variable(self, data=None, shape=None, need_grad=False):
        """A leaf variable; `data` (numpy / torch) is copied into it."""
        if data is not None:
            data = _host(data)
            shape = data.shape
        sh = (ctypes.c_int64 * len(shape))(*[int(s) for s in shape])
        vid = lib().nbg_variable(self._h, len(shape), sh, int(need_grad))
        if vid < 0:
            raise RuntimeError(lib().nbg_last_error().decode())
        v = Var(self, vid)
        if data is not None:
            self.set_data(v, data)
        return v

    def leaf(self, a, shape=None):
        """The leaf variable of parameter array `a` (made at first use), or `a` itself if it is a Var."""
        if isinstance(a, Var):
            return a
        key = (id(a), shape)
        if key not in self._leaves:
            self._keep.append(a)
            h = _host(a)
            self._leaves[key] = self.variable(h.reshape(shape) if shape else h, need_grad=self.need_grad)
        return self._leaves[key]

    def parameter_leaves(self):
        """[(the array passed in, its leaf variable)] in creation order."""
        by_id = {id(a): a for a in self._keep}
        return [(by_id[k[0]], v) for k, v in self._leaves.items()]

    def set_data(self, v, data):
        data = _host(data)
        self._check(lib().nbg_set_data(self._h, v.id, data.ctypes.data_as(ctypes.c_void_p)))

    def shape(self, v):
        sh = (ctypes.c_int64 * 8)()
        nd = ctypes.c_int(0)
        self._check(lib().nbg_shape(self._h, v.id, sh, ctypes.byref(nd)))
        return tuple(int(sh[i]) for i in range(nd.value))

    def data(self, v):
        out = np.empty(self.shape(v), np.float32)
        self._check(lib().nbg_get_data(self._h, v.id, out.ctypes.data_as(ctypes.c_void_p)))
        return out

    def set_persistent(self, v, flag=True):
        self._check(lib().nbg_set_persistent(self._h, v.id, int(flag)))

    # ---- execution -------------------------------------------------------------------
    def forward(self, v, clear_buffer=True, repeat=1):
        """CgVariable::forward `repeat` times; returns seconds per pass (device work included)."""
        sec = ctypes.c_double(0.0)
        self._check(lib().nbg_forward(self._h, v.id, int(clear_buffer), int(repeat), ctypes.byref(sec)))
        return sec.value

    def backward(self, v, grad=None, clear_buffer=True):
        """CgVariable::backward from `v` with initial gradient `grad` (host array of v's shape); returns
        seconds. Leaf gradients accumulate: zero_grad() them first."""
        sec = ctypes.c_double(0.0)
        g = None if grad is None else _host(grad)
        self._check(lib().nbg_backward(self._h, v.id, None if g is None else g.ctypes.data_as(ctypes.c_void_p),
                                       int(clear_buffer), ctypes.byref(sec)))
        return sec.value

    def zero_grad(self, v):
        self._check(lib().nbg_zero_grad(self._h, v.id))

    def grad(self, v):
        out = np.empty(self.shape(v), np.float32)
        self._check(lib().nbg_get_grad(self._h, v.id, out.ctypes.data_as(ctypes.c_void_p)))
        return out

    def profile(self, v, clear_buffer=True, capacity=512):
        """[(function name, ms)] of one forward pass, the device synchronised around every function."""
        names = ctypes.create_string_buffer(64 * capacity)
        ms = (ctypes.c_double * capacity)()
        n = ctypes.c_int(0)
        self._check(lib().nbg_profile(self._h, v.id, int(clear_buffer), names, ms, capacity, ctypes.byref(n)))
        cnt = min(n.value, capacity)
        return [(names.raw[64 * i:64 * i + 64].split(b"\0", 1)[0].decode(), ms[i]) for i in range(cnt)]

    # ---- functions -------------------------------------------------------------------
    def function(self, op, scalars, ivecs, inputs, n_out=1):
        s = (ctypes.c_double * max(1, len(scalars)))(*[float(v) for v in scalars])
        flat = [int(v) for vec in ivecs for v in vec]
        iv = (ctypes.c_int32 * max(1, len(flat)))(*flat)
        ivl = (ctypes.c_int32 * max(1, len(ivecs)))(*[len(v) for v in ivecs])
        ids = (ctypes.c_int32 * len(inputs))(*[v.id for v in inputs])
        outs = (ctypes.c_int32 * n_out)()
        self._check(lib().nbg_function(self._h, op.encode(), s, len(scalars), iv, ivl, len(ivecs), ids, len(inputs),
                                       n_out, outs))
        res = [Var(self, int(o)) for o in outs]
        return res[0] if n_out == 1 else res

    def convolution(self, x, w, b=None, base_axis=1, pad=None, stride=None, dilation=None, group=1,
                    channel_last=False, **kw):
        ins = [self.leaf(x), self.leaf(w)] + ([self.leaf(b)] if b is not None else [])
        return self.function("Convolution", [base_axis, group, channel_last],
                             [pad or (0, 0), stride or (1, 1), dilation or (1, 1)], ins)

    def binary_weight_convolution(self, x, w, wb, alpha, b=None, base_axis=1, pad=None, stride=None, dilation=None,
                                  group=1, quantize_zero_to=1.0, **kw):
        ins = [self.leaf(x), self.leaf(w), self.leaf(wb), self.leaf(alpha)] + ([self.leaf(b)] if b is not None else [])
        return self.function("BinaryWeightConvolution", [base_axis, group, quantize_zero_to],
                             [pad or (0, 0), stride or (1, 1), dilation or (1, 1)], ins)

    def affine(self, x, w, b=None, base_axis=1, **kw):
        ins = [self.leaf(x), self.leaf(w)] + ([self.leaf(b)] if b is not None else [])
        return self.function("Affine", [base_axis], [], ins)

    def batch_normalization(self, x, beta, gamma, mean, var, axes=(1,), decay_rate=0.9, eps=1e-5, batch_stat=True,
                            output_stat=False):
        # the statistics are shaped like x with 1 everywhere but the axis (batch_normalization.cpp:60-90)
        x = self.leaf(x)
        sh = [1] * len(x.shape)
        sh[axes[0]] = x.shape[axes[0]]
        sh = tuple(sh)
        ins = [x] + [self.leaf(a, sh) for a in (beta, gamma, mean, var)]
        return self.function("BatchNormalization", [decay_rate, eps, batch_stat, False, False], [list(axes)], ins)

    def relu(self, x, inplace=False):
        return self.function("ReLU", [False], [], [self.leaf(x)])

    def add2(self, a, b, inplace=False):
        return self.function("Add2", [False], [], [self.leaf(a), self.leaf(b)])

    def fixed_point_quantize(self, x, sign=True, n=8, delta=2 ** -4, quantize=True, ste_fine_grained=True):
        return self.function("FixedPointQuantize", [sign, n, delta, ste_fine_grained], [], [self.leaf(x)])

    def max_pooling(self, x, kernel, stride=None, ignore_border=True, pad=None, channel_last=False):
        return self.function("MaxPooling", [ignore_border, channel_last], [kernel, stride or kernel, pad or (0, 0)],
                             [self.leaf(x)])

    def global_average_pooling(self, x):
        return self.function("GlobalAveragePooling", [], [], [self.leaf(x)])


class Communicator:
    """nnabla's MultiProcessDataParallelCommunicator as registered for `backend` (one process per
    GPU; ranks from RANK / WORLD_SIZE / LOCAL_RANK). Collectives take and return numpy arrays, which
    travel through nnabla's NdArray machinery to the device and back."""
    ALL_REDUCE, REDUCE, BCAST, ALL_GATHER, REDUCE_SCATTER, CALLBACK = range(6)

    def __init__(self, backend="b200:float", device_id="0"):
        L = lib()
        L.nbc_create.restype = ctypes.c_void_p
        L.nbc_last_error.restype = ctypes.c_char_p
        self._h = ctypes.c_void_p(L.nbc_create(backend.encode(), str(device_id).encode()))
        if not self._h:
            raise RuntimeError(L.nbc_last_error().decode())

    def _check(self, rc):
        if rc != 0:
            raise RuntimeError(lib().nbc_last_error().decode())

    def init(self):
        self._check(lib().nbc_init(self._h))

    @property
    def rank(self):
        return lib().nbc_rank(self._h)

    @property
    def size(self):
        return lib().nbc_size(self._h)

    def barrier(self):
        self._check(lib().nbc_barrier(self._h))

    def new_group(self, name, ranks):
        arr = (ctypes.c_int32 * len(ranks))(*ranks)
        self._check(lib().nbc_new_group(self._h, name.encode(), arr, len(ranks)))

    def _run(self, op, arrays, root=0, division=False, inplace=False, group="world"):
        bufs = [np.ascontiguousarray(a, np.float32).copy() for a in arrays]
        ptrs = (ctypes.POINTER(ctypes.c_float) * len(bufs))(*[b.ctypes.data_as(ctypes.POINTER(ctypes.c_float)) for b in bufs])
        sizes = (ctypes.c_int64 * len(bufs))(*[b.size for b in bufs])
        self._check(lib().nbc_collective(self._h, op, ptrs, sizes, len(bufs), int(root), int(division), int(inplace),
                                         group.encode()))
        return bufs

    def all_reduce(self, arrays, division=False, inplace=False, group="world"):
        return self._run(self.ALL_REDUCE, arrays, 0, division, inplace, group)

    def reduce(self, arrays, dst, division=False, inplace=False, group="world"):
        return self._run(self.REDUCE, arrays, dst, division, inplace, group)

    def bcast(self, arrays, src, inplace=False, group="world"):
        return self._run(self.BCAST, arrays, src, False, inplace, group)

    def all_gather(self, array, group="world", n=None):
        n = self.size if n is None else n
        out = self._run(self.ALL_GATHER, [array] + [np.zeros_like(array)] * n, group=group)
        return out[1:]

    def reduce_scatter(self, arrays, division=False, group="world"):
        return self._run(self.REDUCE_SCATTER, [np.zeros_like(arrays[0])] + list(arrays), 0, division, group=group)[0]

    def all_reduce_packed(self, arrays, pack_size, division=False, group="world"):
        """The all_reduce_callback (gradient buckets of pack_size values), run as at the end of a backward pass."""
        return self._run(self.CALLBACK, arrays, pack_size, division, group=group)

    def close(self):
        if self._h:
            lib().nbc_destroy(self._h)
            self._h = None
