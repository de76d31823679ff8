"""ctypes binding of libnnabla_b200.so (the C ABI declared in include/nnabla_b200.h).

There is no fallback: if the library is missing or a call fails, an exception
is raised. Errors surface as RuntimeError carrying the library's message, the
way nnabla surfaces nbla::Exception through Cython (`except +`).
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libnnabla_b200.so")

c_f32p = ctypes.c_void_p
_lib = None

ERROR_NAMES = {1: "value", 2: "target_specific", 3: "memory", 4: "not_implemented", 5: "device_wait"}


class NB200Error(RuntimeError):
    def __init__(self, code, message):
        super().__init__("nnabla_b200 [%s]: %s" % (ERROR_NAMES.get(code, code), message))
        self.code = code


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                "nnabla_b200: %s is missing. Build it with `python -m nnabla_b200.build` "
                "(needs nvcc); there is no CPU or PyTorch fallback." % LIB_PATH)
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.nb200_last_error.restype = ctypes.c_char_p
    return _lib


_calls = 0
_entry = {}  # entry-point name -> ctypes function with its return type set


def calls_made():
    """Number of entry-point calls made through call() so far in this process."""
    return _calls


def call(name, *args):
    """Calls entry point `name` and raises NB200Error on a non-zero status."""
    global _calls
    _calls += 1
    fn = _entry.get(name)
    if fn is None:
        fn = getattr(lib(), name)
        fn.restype = ctypes.c_int
        _entry[name] = fn
    rc = fn(*args)
    if rc != 0:
        raise NB200Error(rc, lib().nb200_last_error().decode("utf-8", "replace"))


def ptr(t):
    """Device (or host) address of a torch tensor / numpy array / None as c_void_p."""
    if t is None:
        return ctypes.c_void_p(0)
    if hasattr(t, "data_ptr"):
        return ctypes.c_void_p(t.data_ptr())
    return ctypes.c_void_p(t.ctypes.data)


def stream_ptr(device=None):
    """torch's current stream of `device` (default: the current device) as a raw cudaStream_t."""
    import torch
    index = device.index if (device is not None and hasattr(device, "index")) else device
    if index is None:
        index = torch.cuda.current_device()
    raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    if raw is not None:  # no Stream object is built on this path: it is taken dozens of times per forward pass
        return ctypes.c_void_p(raw(int(index)))
    return ctypes.c_void_p(torch.cuda.current_stream(index).cuda_stream)


class on_device:
    """`with on_device(dev):` makes `dev` the current CUDA device for the block; when it already
    is (the common case) nothing is switched, which is much cheaper than torch.cuda.device."""
    __slots__ = ("index", "prev")

    def __init__(self, device):
        self.index = device.index if hasattr(device, "index") else device
        self.prev = None

    def __enter__(self):
        import torch
        if self.index is not None:
            cur = torch.cuda.current_device()
            if cur != self.index:
                self.prev = cur
                torch.cuda.set_device(self.index)
        return self

    def __exit__(self, *exc):
        if self.prev is not None:
            import torch
            torch.cuda.set_device(self.prev)
        return False


def i64_array(values):
    return (ctypes.c_int64 * max(1, len(values)))(*[int(v) for v in values])


def i32_array(values):
    return (ctypes.c_int32 * max(1, len(values)))(*[int(v) for v in values])


def size_t(v):
    return ctypes.c_size_t(int(v))


def c_float(v):
    return ctypes.c_float(float(v))
