"""Loader for tests/golden/golden.npz (made by tests/golden/make_golden.py from
the reference's compiled CPU functions)."""
import hashlib
import os

import numpy as np

_G = None


def golden():
    global _G
    if _G is None:
        _G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden.npz"))
    return _G


_GB = None


def golden_backward():
    """tests/golden/golden_backward.npz (made by tests/golden/make_golden_backward.py)."""
    global _GB
    if _GB is None:
        _GB = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_backward.npz"))
    return _GB


def sha(a):
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(a, np.float32).tobytes()).digest(), np.uint8)


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)
