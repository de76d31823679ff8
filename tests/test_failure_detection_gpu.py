"""The give-up path of the bounded device-side waits, run on purpose in the one harmless way:
a one-block kernel waits on a barrier nobody arrives at with a limit of about a millisecond,
returns by itself and leaves its code in the per-device status word. Nothing traps or faults;
the context stays usable and the next contraction on it is correct."""
import ctypes

import numpy as np
import pytest
import torch

from golden_util import bits
from oracle import oracle

pytestmark = pytest.mark.gpu


def test_wait_that_runs_out_is_reported_once_and_the_context_stays_usable():
    from nnabla_b200 import _capi as C
    from nnabla_b200 import functions as F
    torch.cuda.set_device(0)
    C.call("nb200_check_device")
    F.check_device_status()  # clean to start with
    waited = ctypes.c_int(-1)
    C.call("nb200_selftest_wait_timeout", 1000, ctypes.byref(waited), C.stream_ptr())
    # the second role left through the abort flag soon after the first role's 1 ms ran out,
    # not after its own (seconds-long) limit
    assert 900 <= waited.value < 200000, waited.value
    with pytest.raises(C.NB200Error, match="0x101"):   # producer-timeout code
        F.check_device_status()
    F.check_device_status()  # reading the word cleared it
    # the same context runs a contraction correctly afterwards
    rng = np.random.RandomState(0)
    xa = oracle.fixed_point_quantize(rng.randn(64, 256).astype(np.float32), True, 8, 2.0 ** -5)
    wa = oracle.fixed_point_quantize((0.02 * rng.randn(256, 192)).astype(np.float32), True, 8, 2.0 ** -10)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a, np.float32)).cuda()
    y = F.affine(dev(xa), dev(wa), None, fixed_point=(2.0 ** -5, 2.0 ** -10)).cpu().numpy()
    assert np.array_equal(bits(y), bits(oracle.affine(xa, wa, None)))
    F.check_device_status()
    with pytest.raises(C.NB200Error):
        C.call("nb200_selftest_wait_timeout", 0, None, C.stream_ptr())
