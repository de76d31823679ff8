"""Layers with BatchNormalization folded in (the folded graph of nnabla's converter,
python/src/nnabla/experimental/graph_converters/batch_normalization_folding.py:92-200), run as one
kernel per convolution with Add2 / ReLU / FixedPointQuantize in the epilogue and int8 codes out.

Two checks per case:
 * EXACT: the kernel's arithmetic (exact integer accumulation, then one fused multiply-add per step,
   with the factor 2 / delta folded into its constants) restated in numpy on the oracle's exact
   integer convolution: codes bit for bit;
 * against the folded graph on the oracle (Convolution with the folded fp32 weights, Add2, ReLU,
   FixedPointQuantize as separate functions): a fp32 convolution rounds where the integer one does
   not, so a value within that rounding of a quantizer tie may land one step away: codes agree up
   to a small rate of one-step differences."""
import numpy as np
import pytest
import torch

import cases
from golden_util import bits
from nnabla_b200 import resnet18
from oracle import ops as oracle_ops
from oracle import oracle

pytestmark = pytest.mark.gpu
DELTA = 2.0 ** -4


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).cuda()


@pytest.fixture(scope="module")
def F():
    from nnabla_b200 import _capi, functions
    _capi.call("nb200_check_device")
    return functions


def to_codes(y, delta, slots):
    """NCHW multiples of delta -> int8 [batch, pixels, slots] (group 1)."""
    n, c = y.shape[:2]
    k = np.rint(y.reshape(n, c, -1).astype(np.float64) / delta).astype(np.int64)
    assert np.abs(k).max() <= 127
    out = np.zeros((n, k.shape[2], slots), np.int8)
    out[:, :, :c] = k.transpose(0, 2, 1)
    return out


def from_nhwc(a, shape):
    n, c, h, w = shape
    return np.ascontiguousarray(a[:, :, :c].reshape(n, h, w, c).transpose(0, 3, 1, 2))


def quant_codes(v, relu, sign, n, delta):
    """Codes of FixedPointQuantize(relu ? max(v, 0) : v), from the oracle's quantizer."""
    if relu:
        v = oracle.relu(v)
    return np.rint(oracle.fixed_point_quantize(v, sign, n, delta).astype(np.float64) / delta).astype(np.int64)


CASES = [
    # x shape, outmaps, kernel, pad, stride, dilation
    ((2, 64, 14, 14), 64, 3, 1, 1, 1),
    ((3, 64, 12, 12), 128, 3, 1, 2, 1),
    ((2, 64, 12, 12), 128, 1, 0, 2, 1),
    ((2, 128, 10, 10), 128, 3, 1, 1, 1),
    ((2, 256, 7, 7), 512, 3, 1, 1, 1),
    ((5, 512, 7, 7), 512, 3, 1, 1, 1),
    ((1, 48, 9, 11), 80, 3, 1, 1, 1),     # channels and maps that fill neither a K block nor a 32-map chunk
    ((2, 20, 13, 9), 24, 3, 0, 1, 2),     # dilation, no padding
    ((1, 160, 6, 6), 200, 1, 0, 1, 1),
    ((1, 64, 56, 56), 64, 3, 1, 1, 1),    # boxes of two output rows
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "%sx%d-k%d-s%d" % ("x".join(map(str, c[0])), c[1], c[2], c[4]))
@pytest.mark.parametrize("mode", ["plain", "res_codes", "res_float", "float_out", "signed_no_relu"])
def test_folded_convolution(F, case, mode):
    xs, ko, k, pad, stride, dil = case
    rng = np.random.RandomState(ko + k + xs[1])
    xq = oracle.fixed_point_quantize(np.maximum(rng.randn(*xs), 0).astype(np.float32) * 2, True, 8, DELTA)
    if mode == "signed_no_relu":
        xq = oracle.fixed_point_quantize((rng.randn(*xs) * 2).astype(np.float32), True, 8, DELTA)
    w = (rng.randn(ko, xs[1], k, k) * 0.1).astype(np.float32)
    bn = [(0.1 * rng.randn(ko)).astype(np.float32), (1 + 0.1 * rng.randn(ko)).astype(np.float32),
          (0.1 * rng.randn(ko)).astype(np.float32), (0.5 + rng.rand(ko)).astype(np.float32)]
    fold = resnet18.fold_batch_normalization({"l/beta": bn[0], "l/gamma": bn[1], "l/mean": bn[2], "l/var": bn[3]})
    c0, c1 = fold["l"]
    prep = F.prepare_binary_weights(dev(w), 1, 1.0)
    alpha = prep.alpha.cpu().numpy()
    scale = (alpha * c0).astype(np.float32) * np.float32(DELTA)
    slots_in, slots_out = F.codes_nhwc_slots(xs[1]), F.codes_nhwc_slots(ko)
    x_codes = torch.from_numpy(to_codes(xq, DELTA, slots_in)).cuda()
    relu = mode != "signed_no_relu"
    want_shape = oracle.conv_out_shape(xs, w.shape, (pad, pad), (stride, stride), (dil, dil))
    kw = dict(relu=relu)
    res = None
    if mode == "res_codes":
        res = oracle.fixed_point_quantize((rng.randn(*want_shape) * 2).astype(np.float32), True, 8, 2 * DELTA)
        kw.update(residual_codes=torch.from_numpy(to_codes(res, 2 * DELTA, slots_out)).cuda(), residual_delta=2 * DELTA)
    elif mode == "res_float":
        res = rng.randn(*want_shape).astype(np.float32)
        nhwc = np.zeros((want_shape[0], want_shape[2] * want_shape[3], slots_out), np.float32)
        nhwc[:, :, :ko] = res.reshape(want_shape[0], ko, -1).transpose(0, 2, 1)
        kw.update(residual=dev(nhwc))
    elif mode == "float_out":
        kw.update(output="float", relu=False)
    got, shape = F.convolution_codes_folded(x_codes, xs, prep, dev(scale), dev(c1), (pad, pad), (stride, stride),
                                            (dil, dil), **kw)
    F.check_device_status()
    assert tuple(shape) == tuple(want_shape)
    got = got.cpu().numpy()
    assert not got[:, :, ko:].any()  # padding slots stay zero
    # ---- exact restatement: integer accumulator, then the epilogue's rounded operations
    wb = oracle.sign(w, 1.0)
    assert np.array_equal(bits(prep.binary_weight.cpu().numpy()), bits(wb))
    acc = oracle.convolution(np.rint(xq / DELTA).astype(np.float32), wb, None, (pad, pad), (stride, stride),
                             (dil, dil), f64=True)
    assert np.array_equal(acc, np.rint(acc)) and np.abs(acc).max() < 2 ** 24
    # fused multiply-adds in float64 (the products are exact there), rounded once to float32
    fma = lambda a, b, c: (np.asarray(a, np.float64) * np.asarray(b, np.float64) + np.asarray(c, np.float64)).astype(np.float32)
    f = np.float32(1.0 if mode == "float_out" else 2.0 / DELTA)  # codes: u is twice the quantizer's argument
    u = fma(acc, (scale * f).reshape(1, -1, 1, 1), (c1 * f).reshape(1, -1, 1, 1))
    if mode == "res_codes":
        u = fma(np.rint(res / (2 * DELTA)), np.float32(2 * DELTA) * f, u)
    elif mode == "res_float":
        u = fma(res, f, u)
    if mode == "float_out":
        assert np.array_equal(bits(from_nhwc(got, shape)), bits(u))
        return
    cap = np.float32(2 * 127 + 0.5)
    if relu:
        want_exact = (np.floor(np.minimum(np.maximum(u, 0), cap)).astype(np.int64) + 1) >> 1
    else:
        m = (np.floor(np.minimum(np.abs(u), cap)).astype(np.int64) + 1) >> 1
        want_exact = np.where(u < 0, np.maximum(-m, -127), m)
    assert np.array_equal(from_nhwc(got, shape).astype(np.int64), want_exact)
    # ---- the folded graph on the oracle: fp32 convolution with folded weights, then the separate functions
    wal = oracle_ops.binarize(w)[1]
    wf = (c0.reshape(-1, 1, 1, 1) * (wb * wal.reshape(-1, 1, 1, 1))).astype(np.float32)
    ref = oracle.convolution(xq, wf, c1, (pad, pad), (stride, stride), (dil, dil))
    if res is not None:
        ref = oracle.add2(ref, res)
    want = quant_codes(ref, relu, True, 8, DELTA)
    diff = np.abs(from_nhwc(got, shape).astype(np.int64) - want)
    assert diff.max() <= 1 and (diff != 0).mean() < 2e-3, ((diff != 0).mean(), diff.max())


def test_folded_stem(F):
    rng = np.random.RandomState(4)
    x = rng.randn(3, 3, 64, 96).astype(np.float32)
    w = (rng.randn(64, 3, 7, 7) * np.sqrt(2.0 / 147)).astype(np.float32)
    b = (0.1 * rng.randn(64)).astype(np.float32)
    got, shape = F.convolution_relu_fixed_point_codes(dev(x), dev(w), dev(b), (3, 3), (2, 2), True, True, 8, DELTA)
    F.check_device_status()
    ref = oracle.convolution(x, w, b, (3, 3), (2, 2))
    assert tuple(shape) == ref.shape
    diff = np.abs(from_nhwc(got.cpu().numpy(), shape).astype(np.int64) - quant_codes(ref, True, True, 8, DELTA))
    assert diff.max() <= 1 and (diff != 0).mean() < 1e-3
    # without ReLU: signed codes
    got, _ = F.convolution_relu_fixed_point_codes(dev(x), dev(w), None, (3, 3), (2, 2), False, True, 8, DELTA)
    ref = oracle.convolution(x, w, None, (3, 3), (2, 2))
    diff = np.abs(from_nhwc(got.cpu().numpy(), shape).astype(np.int64) - quant_codes(ref, False, True, 8, DELTA))
    assert diff.max() <= 1 and (diff != 0).mean() < 1e-3
    from nnabla_b200._capi import NB200Error
    with pytest.raises(NB200Error):  # not a few-channel geometry
        F.convolution_relu_fixed_point_codes(dev(rng.randn(1, 64, 8, 8)), dev(rng.randn(64, 64, 3, 3)), None, (1, 1),
                                             (1, 1))


def run_folded_network(F, params, x, classes):
    gp = {k: dev(v) for k, v in params.items()}
    trace = []
    net = resnet18.FoldedRunner(F, gp, trace)
    logits = net(dev(x))
    F.check_device_status()
    return net, trace, logits


def check_folded_trace(F, params, trace, picks):
    """Teacher forcing: every fused layer of the GPU run against the folded graph's functions on
    the oracle, fed with the GPU's own input codes of the picked images."""
    fold = resnet18.fold_batch_normalization(params)
    sel = torch.tensor(picks, device="cuda")
    host = lambda t: t.index_select(0, sel).cpu().numpy()
    worst = 0.0
    for rec in trace:
        L, shape = rec["layer"], (len(picks),) + tuple(rec["shape"][1:])
        if L == "stem":
            c0, c1 = fold["stem/bn"]
            ref = oracle.convolution(host(rec["input"]), (c0.reshape(-1, 1, 1, 1) * params["stem/conv/W"]).astype(np.float32),
                                     c1, (3, 3), (2, 2))
            want = quant_codes(ref, True, True, 8, DELTA)
        elif L == "stem/pool":
            xin = from_nhwc(host(rec["input"]), (len(picks),) + tuple(rec["in_shape"][1:])).astype(np.float32) * DELTA
            want = np.rint(oracle.max_pooling(xin, (3, 3), (2, 2), True, (1, 1)) / DELTA).astype(np.int64)
        else:
            k, st = rec["k"], rec["stride"]
            bn = L.replace("conv1", "bn1").replace("conv2", "bn2").replace("shortcut", "bn_s")
            c0, c1 = fold[bn]
            wb, al = oracle_ops.binarize(params[L + "/W"])
            wf = (c0.reshape(-1, 1, 1, 1) * (wb * al.reshape(-1, 1, 1, 1))).astype(np.float32)
            xin = from_nhwc(host(rec["input"]), (len(picks),) + tuple(rec["in_shape"][1:])).astype(np.float32) * DELTA
            ref = oracle.convolution(xin, wf, c1, (k // 2, k // 2), (st, st))
            if L.endswith("shortcut"):
                got = from_nhwc(host(rec["output"]), shape)
                err = cases.rel_rms(got, ref)
                assert err < 1e-5, (L, err)
                continue
            if "residual" in rec:
                ref = oracle.add2(ref, from_nhwc(host(rec["residual"]), shape))
            elif "residual_codes" in rec:
                ref = oracle.add2(ref, from_nhwc(host(rec["residual_codes"]), shape).astype(np.float32) * DELTA)
            want = quant_codes(ref, True, True, 8, DELTA)
        diff = np.abs(from_nhwc(host(rec["output"]), shape).astype(np.int64) - want)
        rate = float((diff != 0).mean())
        worst = max(worst, rate)
        assert diff.max() <= 1 and rate < 2e-3, (L, rate, diff.max())
    return worst


def test_folded_resnet18_small(F):
    rng = np.random.RandomState(0)
    params = resnet18.init_parameters(rng, num_classes=100)
    x = rng.randn(2, 3, 64, 64).astype(np.float32)
    net, trace, logits = run_folded_network(F, params, x, 100)
    assert len(trace) == 2 + 19
    worst = check_folded_trace(F, params, trace, [0, 1])
    net.trace = None
    assert torch.equal(net(dev(x)), logits)  # deterministic
    logits = logits.cpu().numpy()
    ref = resnet18.folded_reference(oracle_ops, params, x, oracle_ops.binarize)
    err = cases.rel_rms(logits, ref)
    gz = lambda w, shape=None: torch.zeros(shape or tuple(w.shape), device="cuda")
    unfolded = resnet18.Runner(F, {k: dev(v) for k, v in params.items()}, gz)(dev(x)).cpu().numpy()
    print("folded ResNet-18 (small): worst per-layer one-step rate %.3g; logits rel-RMS vs the folded oracle graph "
          "%.3g, vs the unfolded GPU graph %.3g" % (worst, err, cases.rel_rms(logits, unfolded)))
    assert err < 2e-2


def test_folded_resnet18_benchmark_size(F):
    rng = np.random.RandomState(0)
    params = resnet18.init_parameters(rng)
    x = rng.randn(256, 3, 224, 224).astype(np.float32)
    net, trace, logits = run_folded_network(F, params, x, 1000)
    picks = [0, 255]
    worst = check_folded_trace(F, params, trace, picks)
    del trace[:]
    logits = logits.cpu().numpy()
    assert logits.shape == (256, 1000) and np.isfinite(logits).all()
    ref = resnet18.folded_reference(oracle_ops, params, x[picks], oracle_ops.binarize)
    err = cases.rel_rms(logits[picks], ref)
    gz = lambda w, shape=None: torch.zeros(shape or tuple(w.shape), device="cuda")
    unfolded = resnet18.Runner(F, {k: dev(v) for k, v in params.items()}, gz, fused="codes")(dev(x)).cpu().numpy()
    agree = float((logits.argmax(1) == unfolded.argmax(1)).mean())
    print("folded ResNet-18 [256,3,224,224]: worst per-layer one-step rate %.3g; logits rel-RMS vs the folded oracle "
          "graph (2 images) %.3g; vs the unfolded GPU graph %.3g, top-1 agreement with it %.3f"
          % (worst, err, cases.rel_rms(logits, unfolded), agree))
    assert err < 2e-2 and agree > 0.9


def test_converter_gives_the_hand_written_folded_network(F):
    """The recorded-graph converter (nnabla_b200/graph_converters.py) applied to the network's own code
    emits the same calls with the same constants as the hand-written FoldedRunner: identical logits."""
    from nnabla_b200 import graph_converters as gc
    rng = np.random.RandomState(8)
    params = resnet18.init_parameters(rng, num_classes=32)
    x = rng.randn(3, 3, 64, 64).astype(np.float32)
    gp = {k: dev(v) for k, v in params.items()}
    rec = gc.Recorder()
    out = resnet18.Runner(rec, gp, lambda w, shape=None: None, None, fixed_point_hint=False)(rec.input)
    prog = gc.BatchNormalizationFolding().convert(rec, out, F)
    assert prog.calls.count("convolution_codes_folded") == 19
    got = prog(dev(x))
    F.check_device_status()
    want = resnet18.FoldedRunner(F, gp)(dev(x))
    assert torch.equal(got, want)


def test_fusion_converter_gives_the_as_written_logits(F):
    """FusedBatchNormalization converter on the recorded network: 17 fused activation calls, every binary-weight
    convolution told the quantizer's step; logits identical to the graph as written and to the hand-written
    Runner(fused=True), bit for bit."""
    from nnabla_b200 import graph_converters as gc
    rng = np.random.RandomState(9)
    params = resnet18.init_parameters(rng, num_classes=32)
    x = rng.randn(3, 3, 64, 64).astype(np.float32)
    gp = {k: dev(v) for k, v in params.items()}
    gz = lambda w, shape=None: torch.zeros(shape if shape is not None else tuple(w.shape), device="cuda")
    rec = gc.Recorder()
    out = resnet18.Runner(rec, gp, lambda w, shape=None: None, None, fixed_point_hint=False)(rec.input)
    prog = gc.FusedBatchNormalization().convert(rec, out, F, gz)
    assert prog.calls.count("bn_add_relu_fixed_point") == 17 and len(prog.calls) == 40
    got = prog(dev(x))
    F.check_device_status()
    as_written = resnet18.Runner(F, gp, gz)(dev(x))
    by_hand = resnet18.Runner(F, gp, gz, fused=True)(dev(x))
    assert torch.equal(got, as_written) and torch.equal(got, by_hand)
