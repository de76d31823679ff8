"""Binary-weight ResNet-18 (BASELINE configs[4]) at a reduced size: every
function of the GPU run is checked against the oracle fed with the GPU's own
inputs (teacher forcing), and the free-running oracle network is compared at
the logits."""
import numpy as np
import pytest
import torch

import cases
import oracle_ops
from golden_util import bits
from oracle import oracle

pytestmark = pytest.mark.gpu


def test_resnet18_per_function_parity_and_logits():
    from nnabla_b200 import functions as F
    from nnabla_b200 import resnet18
    rng = np.random.RandomState(0)
    params = resnet18.init_parameters(rng, num_classes=100)
    x = rng.randn(2, 3, 64, 64).astype(np.float32)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a, np.float32)).cuda()
    gp = {k: dev(v) for k, v in params.items()}
    trace = []
    gz = lambda w, shape=None: torch.zeros(shape or tuple(w.shape), device="cuda")
    net = resnet18.Runner(F, gp, gz, trace)
    logits = net(dev(x)).cpu().numpy()
    F.check_device_status()
    assert logits.shape == (2, 100)
    h = lambda t: t.cpu().numpy()
    exact = {"batch_normalization", "relu", "fixed_point_quantize", "add2", "max_pooling", "global_average_pooling"}
    n_conv = 0
    for rec in trace:
        ins = [h(t) for t in rec["inputs"]]
        got = h(rec["output"])
        L, fn = rec["layer"], rec["fn"]
        if fn == "batch_normalization":
            want = oracle_ops.batch_normalization(ins[0], params[L + "/beta"], params[L + "/gamma"],
                                                  params[L + "/mean"], params[L + "/var"], batch_stat=False)
        elif fn == "relu":
            want = oracle.relu(ins[0])
        elif fn == "fixed_point_quantize":
            want = oracle.fixed_point_quantize(ins[0], True, 8, resnet18.DELTA)
        elif fn == "add2":
            want = oracle.add2(ins[0], ins[1])
        elif fn == "max_pooling":
            want = oracle.max_pooling(ins[0], (3, 3), (2, 2), True, (1, 1))
        elif fn == "global_average_pooling":
            want = oracle.global_average_pooling(ins[0])
        elif fn == "convolution":
            want = oracle.convolution(ins[0], params[L + "/W"], None, (3, 3), (2, 2))
        elif fn == "binary_weight_convolution":
            k, st = rec["attrs"]["k"], rec["attrs"]["stride"]
            want, wwb, wal = oracle.binary_weight_convolution(ins[0], params[L + "/W"], None, (k // 2, k // 2),
                                                              (st, st))
            wb, al = net.side[L]
            assert np.array_equal(bits(h(wb)), bits(wwb)), L
            np.testing.assert_allclose(h(al), wal, rtol=1e-6 + 5000 * 6e-8)
            n_conv += 1
        elif fn == "affine":
            want = oracle.affine(ins[0], params["head/W"], params["head/b"])
        assert got.shape == want.shape, L
        if fn in exact:
            assert np.array_equal(bits(got), bits(want)), "%s (%s) is not bit-exact" % (L, fn)
        else:
            assert cases.rel_rms(got, want) < 1e-5, "%s (%s): %g" % (L, fn, cases.rel_rms(got, want))
    assert n_conv == 19
    # Free-running oracle network: a last-bit difference before a quantizer can move a
    # value by one step, so the logits are compared as a whole, not bit for bit.
    cz = lambda w, shape=None: np.zeros(shape or w.shape, np.float32)
    ref_logits = resnet18.Runner(oracle_ops, params, cz, None, fixed_point_hint=False)(x)
    err = cases.rel_rms(logits, ref_logits)
    print("free-running logits rel-RMS error vs oracle network: %.3g; top-1 agreement: %s"
          % (err, (logits.argmax(1) == ref_logits.argmax(1)).tolist()))
    assert err < 1e-2


def test_macs_per_image_matches_layer_table():
    from nnabla_b200 import resnet18
    assert abs(resnet18.conv_macs_per_image() / 1e6 - 1814) < 10
