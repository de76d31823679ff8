"""The BatchNormalization-folding converter (nnabla_b200/graph_converters.py) on the host: the network is
recorded, matched and turned into a call sequence; a stand-in function namespace notes the calls, so the
matching rules and the folded constants are checked without a GPU."""
import numpy as np
import pytest
import torch

from nnabla_b200 import graph_converters as gc
from nnabla_b200 import resnet18


class FakePrep:
    def __init__(self, w):
        self.alpha = w.abs().mean(dim=(1, 2, 3))
        self.shape, self.group = tuple(w.shape), 1


class FakeOps:
    """Returns placeholders of the right structure and records what it was asked to do."""

    def __init__(self):
        self.log = []

    def prepare_binary_weights(self, w, group, zero_to):
        return FakePrep(w)

    def convolution_relu_fixed_point_codes(self, x, w, b, pad, stride, relu, sign, n, delta):
        self.log.append(("stem", w, b, pad, stride, relu, sign, n, delta))
        return "codes", ("shape",)

    def max_pooling_codes(self, codes, shape, kernel, stride, ib, pad):
        self.log.append(("pool", kernel, stride, ib, pad))
        return "codes", ("shape",)

    def convolution_codes_folded(self, codes, shape, prep, scale, bias, pad, stride, dilation, **kw):
        self.log.append(("conv", prep, scale, bias, pad, stride, kw))
        return ("float" if kw.get("output") == "float" else "codes"), ("shape",)

    def global_average_pooling_codes(self, codes, shape, delta):
        self.log.append(("gap", delta))
        return "pooled"

    def affine(self, x, w, b, base_axis):
        self.log.append(("affine",))
        return "logits"


def record(params):
    rec = gc.Recorder()
    cz = lambda w, shape=None: None
    out = resnet18.Runner(rec, params, cz, None, fixed_point_hint=False)(rec.input)
    return rec, out


def test_resnet18_is_matched_layer_by_layer():
    params = {k: torch.from_numpy(v) for k, v in resnet18.init_parameters(np.random.RandomState(0), 10).items()}
    rec, out = record(params)
    assert len(rec.nodes) == 1 + 3 + 1 + 8 * 9 + 3 * 2 + 2  # stem, its BN/ReLU/quantizer, pool, blocks, shortcuts, head
    ops = FakeOps()
    prog = gc.BatchNormalizationFolding().convert(rec, out, ops)
    assert prog.calls == (["convolution_relu_fixed_point_codes", "max_pooling_codes"]
                          + ["convolution_codes_folded"] * 4                                   # stage 1: no shortcuts
                          + (["convolution_codes_folded"] * 3 + ["convolution_codes_folded"] * 2) * 3
                          + ["global_average_pooling_codes", "affine"])
    assert prog(torch.zeros(1)) == "logits"
    convs = [e for e in ops.log if e[0] == "conv"]
    assert len(convs) == 19
    # the folded constants are those of the hand-written conversion of the same network
    fold = resnet18.fold_batch_normalization(params)
    c0, c1 = fold["stem/bn"]
    stem = ops.log[0]
    assert np.array_equal(stem[1].numpy(), c0.reshape(-1, 1, 1, 1) * params["stem/conv/W"].numpy())
    assert np.array_equal(stem[2].numpy(), c1)
    k0, k1 = fold["stage1/block0/bn1"]
    first = convs[0]
    alpha = params["stage1/block0/conv1/W"].abs().mean(dim=(1, 2, 3)).numpy()
    assert np.array_equal(first[2].numpy(), (alpha * k0).astype(np.float32) * np.float32(resnet18.DELTA))
    assert np.array_equal(first[3].numpy(), k1)
    # stage 1, block 0: conv1 quantizes, conv2 adds the block input as codes
    assert first[6]["relu"] and "residual" not in first[6] and "residual_codes" not in first[6]
    assert convs[1][6]["residual_codes"] == "codes" and convs[1][6]["residual_delta"] == resnet18.DELTA
    # stage 2, block 0: conv1, then the shortcut as fp32 without ReLU, then conv2 with that residual
    s2 = convs[4:7]
    assert s2[0][5] == (2, 2) and s2[1][6].get("output") == "float" and not s2[1][6]["relu"]
    assert s2[2][6]["residual"] == "float" and s2[2][6]["relu"]


def test_what_cannot_be_folded_is_refused():
    w = torch.randn(8, 8, 3, 3)
    bn = [torch.zeros(8), torch.ones(8), torch.zeros(8), torch.ones(8)]
    # a ReLU that no quantizer follows
    rec = gc.Recorder()
    q = rec.fixed_point_quantize(rec.relu(rec.batch_normalization(rec.convolution(rec.input, torch.randn(8, 3, 3, 3)),
                                                                  *bn, batch_stat=False)))
    y = rec.relu(rec.batch_normalization(rec.binary_weight_convolution(q, w, None, None), *bn, batch_stat=False))
    with pytest.raises(NotImplementedError):
        gc.BatchNormalizationFolding().convert(rec, y, FakeOps())
    # training-mode statistics
    rec = gc.Recorder()
    y = rec.fixed_point_quantize(rec.relu(rec.batch_normalization(rec.convolution(rec.input, torch.randn(8, 3, 3, 3)),
                                                                  *bn, batch_stat=True)))
    with pytest.raises(NotImplementedError):
        gc.BatchNormalizationFolding().convert(rec, y, FakeOps())
    # a function outside the folded set
    rec = gc.Recorder()
    y = rec.affine(rec.input, torch.randn(4, 4))
    with pytest.raises(NotImplementedError):
        gc.BatchNormalizationFolding().convert(rec, y, FakeOps())


def test_bias_of_the_convolution_is_folded_too():
    rec = gc.Recorder()
    w, b = torch.randn(8, 3, 3, 3), torch.randn(8)
    bn = [torch.randn(8), torch.rand(8) + 0.5, torch.randn(8), torch.rand(8) + 0.5]
    y = rec.fixed_point_quantize(rec.relu(rec.batch_normalization(rec.convolution(rec.input, w, b, 1, (1, 1)), *bn,
                                                                  batch_stat=False)))
    ops = FakeOps()
    gc.BatchNormalizationFolding().convert(rec, y, ops)(torch.zeros(1))
    beta, gamma, mean, var = [t.numpy() for t in bn]
    std = np.sqrt(var + np.float32(1e-5))
    c0, c1 = gamma / std, beta - gamma * mean / std
    assert np.array_equal(ops.log[0][2].numpy(), c0 * b.numpy() + c1)  # b' = c0 * b + c1


def test_fused_batch_normalization_converter_on_the_oracle():
    """FusedBatchNormalization: 20 BatchNormalization, 8 Add2, 17 ReLU and 17 FixedPointQuantize calls become 17
    fused calls (the three shortcut normalisations join the pass of the block they are added to), everything
    else stays; on the oracle's function namespace the converted program gives the as-written network's
    logits bit for bit (every operation keeps its own rounding)."""
    from oracle import ops as oracle_ops
    rng = np.random.RandomState(3)
    params = resnet18.init_parameters(rng, num_classes=10)
    zeros = lambda w, shape=None: np.zeros(shape if shape is not None else w.shape, np.float32)
    rec = gc.Recorder()
    out = resnet18.Runner(rec, params, zeros, None, fixed_point_hint=False)(rec.input)
    prog = gc.FusedBatchNormalization().convert(rec, out, oracle_ops, zeros)
    assert prog.calls.count("bn_add_relu_fixed_point") == 17 and prog.calls.count("binary_weight_convolution") == 19
    assert not {"batch_normalization", "relu", "add2", "fixed_point_quantize"} & set(prog.calls)
    assert len(prog.calls) == 19 + 17 + 4
    x = rng.randn(1, 3, 32, 32).astype(np.float32)
    want = resnet18.Runner(oracle_ops, params, zeros, None, fixed_point_hint=False)(x)
    got = prog(x)
    assert np.array_equal(np.asarray(got, np.float32).view(np.uint32), np.asarray(want, np.float32).view(np.uint32))


def test_fused_batch_normalization_converter_leaves_other_patterns_alone():
    """A BatchNormalization with nothing to fuse with, one in training mode and one that feeds two functions
    stay plain calls; an Add2 of a tensor with itself is not taken apart."""
    rec = gc.Recorder()
    c = np.ones(4, np.float32).reshape(1, 4, 1, 1)
    a = rec.batch_normalization(rec.input, c, c, c, c, [1], 0.9, 1e-5, False)          # -> max_pooling: plain
    p = rec.max_pooling(a, (2, 2), (2, 2))
    b = rec.batch_normalization(p, c, c, c, c, [1], 0.9, 1e-5, True)                   # batch statistics: plain
    r = rec.relu(b)
    d = rec.batch_normalization(r, c, c, c, c, [1], 0.9, 1e-5, False)                  # two consumers: plain
    e = rec.add2(rec.relu(d), rec.fixed_point_quantize(d))
    f = rec.batch_normalization(e, c, c, c, c, [1], 0.9, 1e-5, False)                  # -> ReLU: fused
    g = rec.relu(f)
    h = rec.add2(g, g)

    class Ops:
        def __getattr__(self, name):
            return lambda *a, **k: name
    prog = gc.FusedBatchNormalization().convert(rec, h, Ops(), None)
    assert prog.calls == ["batch_normalization", "max_pooling", "batch_normalization", "relu", "batch_normalization",
                          "relu", "fixed_point_quantize", "add2", "bn_add_relu_fixed_point", "add2"]
