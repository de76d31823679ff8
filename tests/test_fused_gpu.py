"""The fused BN (+ residual) + ReLU + FixedPointQuantize pass must be
bit-identical to the chain of separate functions (checked against the oracle
chain), and a ResNet-18 that uses it must produce the same logits, bit for
bit, as the unfused network on the same device."""
import numpy as np
import pytest
import torch

import oracle_ops
from golden_util import bits

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).cuda()


@pytest.fixture(scope="module")
def F():
    from nnabla_b200 import _capi, functions
    _capi.call("nb200_check_device")
    return functions


def bn_set(rng, c):
    return [(0.1 * rng.randn(c)).astype(np.float32), (1 + 0.1 * rng.randn(c)).astype(np.float32),
            (0.1 * rng.randn(c)).astype(np.float32), (0.5 + rng.rand(c)).astype(np.float32)]


@pytest.mark.parametrize("shape", [(2, 8, 6, 6), (3, 5, 7, 3), (1, 64, 56, 56), (4, 3, 1, 1)])
@pytest.mark.parametrize("second", ["none", "residual", "bn"])
@pytest.mark.parametrize("delta", [2.0 ** -4, 0.05])
def test_fused_equals_chain(F, shape, second, delta):
    rng = np.random.RandomState(sum(shape))
    a = (rng.randn(*shape) * 3).astype(np.float32)
    b = (rng.randn(*shape) * 3).astype(np.float32) if second != "none" else None
    pa = bn_set(rng, shape[1])
    pb = bn_set(rng, shape[1]) if second == "bn" else None
    want = oracle_ops.bn_add_relu_fixed_point(a, pa, b, pb, 1e-5, True, True, True, 8, delta)
    got = F.bn_add_relu_fixed_point(dev(a), [dev(t) for t in pa], dev(b) if b is not None else None,
                                    [dev(t) for t in pb] if pb else None, 1e-5, True, True, True, 8, delta)
    assert np.array_equal(bits(got.cpu().numpy()), bits(want))


def test_stages_can_be_switched_off(F):
    rng = np.random.RandomState(1)
    a = rng.randn(2, 4, 5, 5).astype(np.float32)
    pa = bn_set(rng, 4)
    want = oracle_ops.bn_add_relu_fixed_point(a, pa, None, None, 1e-5, False, False)
    got = F.bn_add_relu_fixed_point(dev(a), [dev(t) for t in pa], relu=False, quantize=False)
    assert np.array_equal(bits(got.cpu().numpy()), bits(want))
    want = oracle_ops.bn_add_relu_fixed_point(a, pa, None, None, 1e-5, True, False)
    got = F.bn_add_relu_fixed_point(dev(a), [dev(t) for t in pa], relu=True, quantize=False)
    assert np.array_equal(bits(got.cpu().numpy()), bits(want))


def test_fused_resnet_equals_unfused(F):
    from nnabla_b200 import resnet18
    rng = np.random.RandomState(0)
    params = resnet18.init_parameters(rng, num_classes=100)
    x = dev(rng.randn(2, 3, 64, 64).astype(np.float32))
    gp = {k: dev(v) for k, v in params.items()}
    gz = lambda w, shape=None: torch.zeros(shape or tuple(w.shape), device="cuda")
    plain = resnet18.Runner(F, gp, gz)(x)
    fused = resnet18.Runner(F, gp, gz, fused=True)(x)
    F.check_device_status()
    assert torch.equal(plain, fused)
