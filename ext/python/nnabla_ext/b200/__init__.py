"""nnabla extension package for the "b200" backend.

Follows the convention of python/src/nnabla_ext/cpu/__init__.py:17-45 and
doc/python/api/ext.rst:30-60: importing the package registers the backend
(init_b200), and the module exposes context(), synchronize(),
clear_memory_cache(), array_classes(), device_synchronize(),
get_device_count() and get_devices(), which is what
nnabla.ext_utils.get_extension_context('b200', device_id=...),
nnabla.utils.profiler.GraphProfiler and the function benchmark harness call.

It needs the nnabla Python package (Cython bindings over libnnabla), which
cannot be built without nnabla's code generator; until then the same classes
are driven through the C binding of ext/runner (nnabla_b200/nbla_graph.py,
tests/test_ext_gpu.py). The native entry points used below are those of
ext/_build/libnnabla_ext_b200.so.
"""
import ctypes
import os

import nnabla as nn  # noqa: F401  (the host package; absent in this build environment)

_HERE = os.path.dirname(os.path.abspath(__file__))
_lib = ctypes.CDLL(os.environ.get("NNABLA_EXT_B200_LIB", os.path.join(_HERE, "libnnabla_ext_b200.so")),
                   mode=ctypes.RTLD_GLOBAL)
_lib.nnabla_ext_b200_last_error.restype = ctypes.c_char_p
if _lib.nnabla_ext_b200_init() != 0:
    raise ImportError("nnabla_ext.b200: " + _lib.nnabla_ext_b200_last_error().decode())
_nb200_lib = None


def array_classes():
    return ["B200CachedArray", "B200Array"]


def context(device_id="0", type_config="float", **kw):
    """Context of the b200 backend. There is deliberately no 'cpu:float' entry:
    a function without a b200 implementation raises instead of falling back.
    type_config='half' gives ['b200:half', 'b200:float'] as nnabla's extensions do; nothing is registered under
    'b200:half', so the function registry resolves every function to its float implementation."""
    if type_config == "half":
        return nn.Context(["b200:half", "b200:float"], array_classes()[0], str(device_id))
    if type_config != "float":
        raise ValueError("Unknown data type config is given %s" % type_config)
    return nn.Context(["b200:float"], array_classes()[0], str(device_id))


def device_synchronize(device_id="0", **kw):
    if _lib.nnabla_ext_b200_device_synchronize(int(device_id)) != 0:
        raise RuntimeError(_lib.nnabla_ext_b200_last_error().decode())


def synchronize(device_id="0", **kw):
    device_synchronize(device_id)


def clear_memory_cache():
    """Returns the caching allocator's unused device blocks to the driver."""
    if _lib.nnabla_ext_b200_clear_memory_cache() != 0:
        raise RuntimeError(_lib.nnabla_ext_b200_last_error().decode())


def get_device_count():
    n = ctypes.c_int(0)
    _nb200().nb200_device_count(ctypes.byref(n))
    return n.value


def get_devices():
    return [str(i) for i in range(get_device_count())]


def _nb200():
    """The C-ABI library, already mapped as a dependency of the extension library."""
    global _nb200_lib
    if _nb200_lib is None:
        _nb200_lib = ctypes.CDLL(os.environ.get("NNABLA_B200_LIB", "libnnabla_b200.so"))
    return _nb200_lib
