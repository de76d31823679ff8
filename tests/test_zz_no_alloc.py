"""The allocation-free min-max quantizer entry point against the regular one.

Some hosts cannot let a library allocate device memory: frameworks whose own
allocator owns the whole device (nnabla's caching allocator works that way)
and serving loops that must not take the driver's allocation locks. For them
nb200_min_max_quantize_f32_noalloc keeps its scratch in a fixed array inside
the library. This file checks, through the C ABI, that it returns exactly what
nb200_min_max_quantize_f32 returns, on two calls in a row (the second call
finds the first call's leftovers in the shared array), and that it refuses
more ranges than the array holds. It is named to be collected last.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(entry, x, qmin, qmax, lmin, lmax, decay, x_min_max, ema, eps):
    from nnabla_b200 import _capi as C
    y = torch.empty_like(x)
    scale = torch.empty_like(qmin)
    C.call(entry, C.ptr(x), C.i64_array(x.shape), x.dim(), C.ptr(qmin), C.ptr(qmax), C.ptr(lmin), C.ptr(lmax),
           C.i64_array(qmin.shape), C.c_float(decay), int(x_min_max), int(ema), C.c_float(eps), C.ptr(y),
           C.ptr(scale), C.stream_ptr(x.device))
    torch.cuda.synchronize()
    return y, scale


def _inputs(seed, x_shape, q_shape):
    rng = np.random.RandomState(seed)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a, np.float32)).cuda()
    return (t(rng.randn(*x_shape) * 2), t(-0.5 * rng.rand(*q_shape)), t(0.5 * rng.rand(*q_shape)),
            t(np.zeros(q_shape)), t(np.full(q_shape, 255.0)))


def test_noalloc_matches_regular_entry_point_twice():
    from nnabla_b200 import _capi as C
    torch.cuda.set_device(0)
    C.call("nb200_check_device")
    # call 1: per-channel ranges with the moving-average update (uses every scratch slot);
    # call 2: fewer ranges, given min/max (the min/max slots still hold call 1's values).
    plan = [(1, (4, 8, 16, 16), (1, 8, 1, 1), 0.9, True, True),
            (2, (16, 8, 3, 3), (16, 1, 1, 1), 0.999, False, False),
            (3, (1 << 16,), (1,), 0.999, True, False)]
    for seed, xs, qs, decay, xmm, ema in plan:
        x, qmin, qmax, lmin, lmax = _inputs(seed, xs, qs)
        rmin, rmax = qmin.clone(), qmax.clone()
        want_y, want_s = _call("nb200_min_max_quantize_f32", x, rmin, rmax, lmin, lmax, decay, xmm, ema, 0.01)
        nmin, nmax = qmin.clone(), qmax.clone()
        got_y, got_s = _call("nb200_min_max_quantize_f32_noalloc", x, nmin, nmax, lmin, lmax, decay, xmm, ema, 0.01)
        # integer/bit work: the two entry points run the same kernels, so the match is exact
        assert torch.equal(got_y.view(torch.int32), want_y.view(torch.int32))
        assert torch.equal(got_s.view(torch.int32), want_s.view(torch.int32))
        assert torch.equal(nmin.view(torch.int32), rmin.view(torch.int32))
        assert torch.equal(nmax.view(torch.int32), rmax.view(torch.int32))


def _pool_high(reset):
    from nnabla_b200 import _capi as C
    high = ctypes.c_int64(0)
    C.call("nb200_scratch_pool_stats", None, ctypes.byref(high), int(reset))
    return high.value


def test_noalloc_takes_nothing_from_the_scratch_pool():
    """What the entry point is for: between a reset of the scratch pool's high-water mark and the
    end of the call the mark does not move, while the regular entry point (which takes its 28 bytes
    per range from the pool) moves it. torch's own allocator is not involved in either call: every
    tensor is made before the mark is reset."""
    from nnabla_b200 import _capi as C
    torch.cuda.set_device(0)
    x, qmin, qmax, lmin, lmax = _inputs(5, (4, 8, 16, 16), (1, 8, 1, 1))
    y, scale = torch.empty_like(x), torch.empty_like(qmin)

    def run(entry):
        C.call(entry, C.ptr(x), C.i64_array(x.shape), x.dim(), C.ptr(qmin), C.ptr(qmax), C.ptr(lmin), C.ptr(lmax),
               C.i64_array(qmin.shape), C.c_float(0.9), 1, 1, C.c_float(0.01), C.ptr(y), C.ptr(scale),
               C.stream_ptr(x.device))
        torch.cuda.synchronize()
    run("nb200_min_max_quantize_f32_noalloc")  # first call on the device: address lookup, tables
    torch.cuda.synchronize()
    before = _pool_high(reset=True)
    run("nb200_min_max_quantize_f32_noalloc")
    assert _pool_high(reset=False) == before
    before = _pool_high(reset=True)
    run("nb200_min_max_quantize_f32")
    assert _pool_high(reset=False) > before


def test_noalloc_refuses_more_ranges_than_its_array_holds():
    from nnabla_b200 import _capi as C
    torch.cuda.set_device(0)
    x, qmin, qmax, lmin, lmax = _inputs(4, (4097, 2), (4097, 1))
    with pytest.raises(RuntimeError, match="at most 4096"):
        _call("nb200_min_max_quantize_f32_noalloc", x, qmin, qmax, lmin, lmax, 0.999, False, False, 0.01)
    # the regular entry point takes the same call
    _call("nb200_min_max_quantize_f32", x, qmin, qmax, lmin, lmax, 0.999, False, False, 0.01)
