"""The C-ABI library loads on a machine without a GPU and exports every entry
point that include/*.h declares (no compute call is made here)."""
import ctypes
import glob
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = []
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = open(h).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"\b(nb200_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


@pytest.fixture(scope="module")
def library():
    from nnabla_b200 import build
    build.build()
    return ctypes.CDLL(build.LIB)


def test_header_declares_entry_points():
    syms = declared_symbols()
    assert len(syms) >= 20
    for required in ("nb200_fixed_point_quantize_f32", "nb200_pow2_quantize_f32", "nb200_min_max_quantize_f32"):
        assert required in syms


def test_every_declared_symbol_is_exported(library):
    missing = [s for s in declared_symbols() if not hasattr(library, s)]
    assert not missing, "declared in include/*.h but not exported: %s" % missing


def test_error_reporting_without_gpu(library):
    library.nb200_last_error.restype = ctypes.c_char_p
    assert library.nb200_abi_version() >= 1
    # Argument checks run before any CUDA call: the reference's setup errors.
    rc = library.nb200_fixed_point_quantize_f32(None, None, ctypes.c_size_t(0), 1, 0, ctypes.c_float(0.5), None)
    assert rc == 1 and b"positive" in library.nb200_last_error()
    rc = library.nb200_fixed_point_quantize_f32(None, None, ctypes.c_size_t(0), 1, 1, ctypes.c_float(0.5), None)
    assert rc == 1 and b"sign" in library.nb200_last_error()
    rc = library.nb200_pow2_quantize_f32(None, None, ctypes.c_size_t(0), 1, 1, 2, 0, None)
    assert rc == 1 and b"zero" in library.nb200_last_error()


def test_python_mirror_refuses_cpu_tensors():
    import torch
    from nnabla_b200 import functions as F
    with pytest.raises(RuntimeError, match="no CPU path"):
        F.fixed_point_quantize(torch.zeros(4))
    # quantize=False is the identity, as in python/src/nnabla/functions.py:480-482
    x = torch.zeros(4)
    assert F.fixed_point_quantize(x, quantize=False) is x
    assert F.pow2_quantize(x, quantize=False) is x


def test_code_layout_arithmetic_without_gpu(library):
    """Slots per pixel of the int8 channel-last layout and the argument checks of the code chain
    (host arithmetic only: batch 0 returns before any CUDA call)."""
    from nnabla_b200 import functions as F
    library.nb200_last_error.restype = ctypes.c_char_p
    for channels, group, want in ((3, 1, 64), (64, 1, 64), (65, 1, 128), (80, 1, 128), (128, 1, 128), (200, 1, 208),
                                  (256, 1, 256), (48, 3, 64), (96, 2, 96), (512, 4, 512)):
        assert F.codes_nhwc_slots(channels, group) == want, (channels, group)
    with pytest.raises(RuntimeError):
        F.codes_nhwc_slots(10, 3)
    z = ctypes.c_int64(0)
    # 8 unsigned bits do not fit an int8 code; n - sign = 7 does
    rc = library.nb200_bn_add_relu_fxp_codes_nhwc(None, None, None, None, None, None, None, None, None, None, None,
                                                  ctypes.c_float(1.0), None, z, ctypes.c_int64(8), ctypes.c_int64(4), 1,
                                                  ctypes.c_float(1e-5), 1, 0, 8, ctypes.c_float(0.25), None)
    assert rc == 4 and b"int8" in library.nb200_last_error()
    rc = library.nb200_bn_add_relu_fxp_codes_nhwc(None, None, None, None, None, None, None, None, None, None, None,
                                                  ctypes.c_float(1.0), None, z, ctypes.c_int64(8), ctypes.c_int64(4), 1,
                                                  ctypes.c_float(1e-5), 1, 1, 8, ctypes.c_float(0.25), None)
    assert rc == 0
    # pooling: padding must be smaller than the window
    rc = library.nb200_max_pooling_codes_nhwc(None, None, z, ctypes.c_int64(8), 6, 6, 1, 2, 2, 2, 2, 2, 0, 1, None)
    assert rc == 1 and b"padding" in library.nb200_last_error()
