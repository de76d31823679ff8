"""Binary-weight ResNet-18: every function of the GPU run is checked against the
oracle fed with the GPU's own inputs (teacher forcing), and the free-running
oracle network is compared at the logits; once at a reduced size and once at
the benchmark's size (256 x 3 x 224 x 224, 1000 classes), where the oracle
follows two images of the batch."""
import numpy as np
import pytest
import torch

import cases
from oracle import ops as oracle_ops
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


def _want(rec, ins, params):
    """Oracle result of one traced function call on the given (host) inputs."""
    from nnabla_b200 import resnet18
    L, fn = rec["layer"], rec["fn"]
    if fn == "batch_normalization":
        return oracle_ops.batch_normalization(ins[0], params[L + "/beta"], params[L + "/gamma"], params[L + "/mean"],
                                              params[L + "/var"], batch_stat=False)
    if fn == "relu":
        return oracle.relu(ins[0])
    if fn == "fixed_point_quantize":
        return oracle.fixed_point_quantize(ins[0], True, 8, resnet18.DELTA)
    if fn == "add2":
        return oracle.add2(ins[0], ins[1])
    if fn == "max_pooling":
        return oracle.max_pooling(ins[0], (3, 3), (2, 2), True, (1, 1))
    if fn == "global_average_pooling":
        return oracle.global_average_pooling(ins[0])
    if fn == "convolution":
        return oracle.convolution(ins[0], params[L + "/W"], None, (3, 3), (2, 2))
    if fn == "binary_weight_convolution":
        k, st = rec["attrs"]["k"], rec["attrs"]["stride"]
        return oracle.binary_weight_convolution(ins[0], params[L + "/W"], None, (k // 2, k // 2), (st, st))[0]
    if fn == "affine":
        return oracle.affine(ins[0], params["head/W"], params["head/b"])
    raise AssertionError(fn)


def test_resnet18_benchmark_size_all_forms():
    """The benchmark's network at its stated size: input [256, 3, 224, 224] ~ N(0, 1), 1000 classes,
    seed 0. The GPU runs the whole batch (so that every layer takes the tile shapes, pixel boxes and
    store paths of the timed geometry) in four forms: as the graph is written, with the fused
    activation pass, with int8 codes between the layers, and with prepared weights. All four must
    give the same logits bit for bit. The oracle follows images 0 and 255 of the batch (every
    function of this network treats the images independently): teacher-forced per-function checks
    of the as-written run, then the free-running oracle network against the logits, with the
    quantizer flip rate and the top-1 agreement."""
    from nnabla_b200 import functions as F
    from nnabla_b200 import resnet18
    rng = np.random.RandomState(0)
    params = resnet18.init_parameters(rng)
    x = rng.randn(256, 3, 224, 224).astype(np.float32)
    picks = [0, 255]
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a, np.float32)).cuda()
    gp = {k: dev(v) for k, v in params.items()}
    gz = lambda w, shape=None: torch.zeros(shape or tuple(w.shape), device="cuda")
    xd = dev(x)
    trace = []
    net = resnet18.Runner(F, gp, gz, trace)
    logits_d = net(xd)
    F.check_device_status()
    assert tuple(logits_d.shape) == (256, 1000)
    # ---- teacher forcing on the two images --------------------------------------------------
    exact = {"batch_normalization", "relu", "fixed_point_quantize", "add2", "max_pooling", "global_average_pooling"}
    sel = torch.tensor(picks, device="cuda")
    gpu_quant = {}
    n_conv = 0
    for rec in trace:
        ins = [t.index_select(0, sel).cpu().numpy() for t in rec["inputs"]]
        got = rec["output"].index_select(0, sel).cpu().numpy()
        want = _want(rec, ins, params)
        L, fn = rec["layer"], rec["fn"]
        assert got.shape == want.shape, L
        if fn in exact:
            assert np.array_equal(bits(got), bits(want)), "%s (%s) is not bit-exact" % (L, fn)
        else:
            err = cases.rel_rms(got, want)
            assert err < 1e-5, "%s (%s): %g" % (L, fn, err)
        if fn == "fixed_point_quantize":
            gpu_quant[L] = got
        if fn == "binary_weight_convolution":
            wwb = oracle.sign(params[L + "/W"], 1.0)
            assert np.array_equal(bits(net.side[L][0].cpu().numpy()), bits(wwb)), L
            n_conv += 1
    assert n_conv == 19 and len(gpu_quant) == 17
    del trace[:]
    net.trace = None
    # ---- the other three forms: same logits, bit for bit -------------------------------------
    for kw in (dict(fused=True), dict(fused="codes"), dict(fused="codes", prepared_weights=True)):
        other = resnet18.Runner(F, gp, gz, **kw)(xd)
        F.check_device_status()
        assert torch.equal(other, logits_d), kw
        del other
    logits = logits_d.cpu().numpy()
    assert np.isfinite(logits).all()
    # ---- free-running oracle network on the two images ---------------------------------------
    cz = lambda w, shape=None: np.zeros(shape or w.shape, np.float32)
    otrace = []
    ref_logits = resnet18.Runner(oracle_ops, params, cz, otrace, fixed_point_hint=False)(x[picks])
    # A last-bit difference before a quantizer can move a value by one step, and one moved value
    # shifts every output it feeds by alpha * delta, so flips multiply from layer to layer: the
    # rate is asserted where it starts (after the stem) and reported for the whole network.
    rates = []
    flips = total = 0
    for rec in otrace:
        if rec["fn"] == "fixed_point_quantize":
            d = int((bits(rec["output"]) != bits(gpu_quant[rec["layer"]])).sum())
            rates.append((rec["layer"], d / rec["output"].size))
            flips += d
            total += rec["output"].size
            assert np.abs(rec["output"] - gpu_quant[rec["layer"]]).max() <= resnet18.DELTA * (1 + 1e-6) or d == 0 or \
                rec["layer"] != "stem/fxp"
    err = cases.rel_rms(logits[picks], ref_logits)
    agree = (logits[picks].argmax(1) == ref_logits.argmax(1)).tolist()
    print("benchmark-size ResNet-18: free-running logits rel-RMS %.3g; quantizer flip rate: first layer %.3g, "
          "last layer %.3g, all layers %.3g (%d of %d); top-1 agreement %s"
          % (err, rates[0][1], rates[-1][1], flips / total, flips, total, agree))
    assert rates[0][0] == "stem/fxp" and rates[0][1] < 1e-4
    assert err < 1e-2


def test_macs_per_image_matches_layer_table():
    from nnabla_b200 import resnet18
    assert abs(resnet18.conv_macs_per_image() / 1e6 - 1814) < 10
