"""Host-side logic of the extension's communicator that needs no GPU: the bucket plan of the packed
gradient all-reduce, and the registry (the CPU context has no communicator, as in the reference)."""
import ctypes

import pytest

from nnabla_b200 import nbla_graph

pytestmark = pytest.mark.skipif(not nbla_graph.available(), reason="runner library not built")


def plan(sizes, pack):
    L = nbla_graph.lib()
    out = (ctypes.c_int64 * (len(sizes) + 2))()
    n = L.nbc_plan_buckets((ctypes.c_int64 * max(1, len(sizes)))(*sizes), len(sizes), ctypes.c_int64(pack), out,
                           len(sizes) + 2)
    assert n >= 1
    return [int(out[i]) for i in range(n)]


def test_bucket_plan():
    assert plan([], 100) == [0, 0]
    assert plan([10, 20, 30], 100) == [0, 3]
    assert plan([60, 50, 40, 70], 100) == [0, 1, 3, 4]      # 60 | 50 + 40 | 70
    assert plan([500, 1, 1], 100) == [0, 1, 3]               # an array larger than a bucket stands alone
    assert plan([100, 100], 100) == [0, 1, 2]
    sizes = [9408, 64, 64, 64, 64] + [36864, 64] * 8
    p = plan(sizes, 1 << 16)
    assert p[0] == 0 and p[-1] == len(sizes) and all(b > a for a, b in zip(p, p[1:]))
    for a, b in zip(p, p[1:]):
        assert sum(sizes[a:b]) <= (1 << 16) or b - a == 1


def test_cpu_context_has_no_communicator():
    L = nbla_graph.lib()
    L.nbc_create.restype = ctypes.c_void_p
    L.nbc_last_error.restype = ctypes.c_char_p
    h = L.nbc_create(b"cpu:float", b"0")
    assert not h and b"cpu" in L.nbc_last_error().lower()
