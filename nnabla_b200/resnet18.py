"""Binary-weight ResNet-18 on 224 x 224 inputs with 1000 classes, written against the F / PF mirrors.

The reference ships no in-tree definition (python/src/nnabla/models/imagenet/resnet.py:59-60
only loads a downloaded archive); this is the standard 18-layer basic-block
topology: stem convolution 7x7/2 + BN + ReLU + max-pooling 3x3/2, four stages of
two basic blocks with 64/128/256/512 maps and 1x1 stride-2 projection
shortcuts, global average pooling, affine to 1000 classes. The first
convolution and the final affine are full precision; every other convolution
is a BinaryWeightConvolution; FixedPointQuantize(sign, n=8, delta=2^-4)
follows every ReLU; BatchNormalization runs in inference mode on running
statistics.

`ops` is the function namespace (nnabla_b200.functions on the GPU; the tests
pass an oracle-backed namespace with the same names), `params` maps parameter
names to arrays, `trace` (optional list) records every function call for
per-function parity checks.
"""
import numpy as np

DELTA = 2.0 ** -4
STAGES = [(64, 1), (128, 2), (256, 2), (512, 2)]


def init_parameters(rng, num_classes=1000, in_channels=3):
    """Random initialisation (numpy, seeded): Kaiming-normal convolution weights,
    random BN running statistics with var > 0."""
    p = {}

    def conv(name, o, i, k):
        p[name + "/W"] = (rng.randn(o, i, k, k) * np.sqrt(2.0 / (i * k * k))).astype(np.float32)

    def bn(name, c):
        p[name + "/beta"] = (0.1 * rng.randn(c)).astype(np.float32)
        p[name + "/gamma"] = (1.0 + 0.1 * rng.randn(c)).astype(np.float32)
        p[name + "/mean"] = (0.1 * rng.randn(c)).astype(np.float32)
        p[name + "/var"] = (0.5 + rng.rand(c)).astype(np.float32)

    conv("stem/conv", 64, in_channels, 7)
    bn("stem/bn", 64)
    cin = 64
    for s, (c, stride) in enumerate(STAGES):
        for b in range(2):
            st = stride if b == 0 else 1
            name = "stage%d/block%d" % (s + 1, b)
            conv(name + "/conv1", c, cin, 3)
            bn(name + "/bn1", c)
            conv(name + "/conv2", c, c, 3)
            bn(name + "/bn2", c)
            if st != 1 or cin != c:
                conv(name + "/shortcut", c, cin, 1)
                bn(name + "/bn_s", c)
            cin = c
    p["head/W"] = (rng.randn(512, num_classes) * np.sqrt(1.0 / 512)).astype(np.float32)
    p["head/b"] = (0.01 * rng.randn(num_classes)).astype(np.float32)
    return p


class Runner:
    """Applies the network with a given function namespace and array factory."""

    def __init__(self, ops, params, zeros_like, trace=None, fixed_point_hint=True, fused=False,
                 prepared_weights=False, batch_stat=False, codes_sideband=False):
        """fused=True applies BN (+ residual) + ReLU + FixedPointQuantize as one
        function (ops.bn_add_relu_fixed_point), which is bit-identical to the
        separate functions and reads / writes each activation once.
        fused="codes" additionally keeps the quantized activations between the
        binary-weight layers as int8 channel-last codes (1 byte per value, the
        layout the int8 convolution reads; the residual is code * delta): the
        same logits, bit for bit."""
        # prepared_weights (with fused="codes"): binarise every weight once, at its first use,
        # instead of in every forward pass; for inference with weights that do not change
        # batch_stat=True: BatchNormalization uses (and updates) batch statistics, the training graph
        # codes_sideband (graph as written): every FixedPointQuantize also leaves int8 channel-last codes with its
        # result, which the binary-weight convolutions behind it read instead of converting the fp32 tensor again
        self.codes_sideband = codes_sideband
        self.batch_stat = batch_stat
        self.prepared_weights = prepared_weights
        self.prepared = {}
        self.fused = fused
        self.ops = ops
        self.p = params
        self.zeros_like = zeros_like
        self.trace = trace
        self.hint = fixed_point_hint
        self.side = {}  # Wb / alpha buffers, written by the binary layers

    def _rec(self, name, fn, inputs, out, **attrs):
        if self.trace is not None:
            self.trace.append({"layer": name, "fn": fn, "inputs": inputs, "output": out, "attrs": attrs})
        return out

    def bn(self, name, x):
        p = self.p
        y = self.ops.batch_normalization(x, p[name + "/beta"], p[name + "/gamma"], p[name + "/mean"],
                                         p[name + "/var"], [1], 0.9, 1e-5, self.batch_stat)
        return self._rec(name, "batch_normalization", [x], y)

    def relu_q(self, name, x, to_convolution=True):
        y = self._rec(name + "/relu", "relu", [x], self.ops.relu(x))
        kw = {"codes_sideband": True} if self.codes_sideband and to_convolution else {}
        q = self.ops.fixed_point_quantize(y, True, 8, DELTA, **kw)
        return self._rec(name + "/fxp", "fixed_point_quantize", [y], q)

    def bn_params(self, name):
        p = self.p
        return (p[name + "/beta"], p[name + "/gamma"], p[name + "/mean"], p[name + "/var"])

    def fused_act(self, name, a, bn_a, b=None, bn_b=None):
        y = self.ops.bn_add_relu_fixed_point(a, self.bn_params(bn_a), b, self.bn_params(bn_b) if bn_b else None, 1e-5,
                                             True, True, True, 8, DELTA)
        return self._rec(name, "bn_add_relu_fixed_point", [a] + ([b] if b is not None else []), y, bn_a=bn_a,
                         bn_b=bn_b)

    def bwconv(self, name, x, k, stride):
        w = self.p[name + "/W"]
        if name not in self.side:
            self.side[name] = (self.zeros_like(w), self.zeros_like(w, (w.shape[0],)))
        wb, alpha = self.side[name]
        pad = (k // 2, k // 2)
        kw = {"fixed_point_delta": DELTA} if self.hint else {}
        y = self.ops.binary_weight_convolution(x, w, wb, alpha, None, 1, pad, (stride, stride), (1, 1), 1, 1.0, **kw)
        return self._rec(name, "binary_weight_convolution", [x], y, k=k, stride=stride)

    def bwconv_codes(self, name, codes, shape, k, stride):
        w = self.p[name + "/W"]
        if self.prepared_weights:
            if name not in self.prepared:
                self.prepared[name] = self.ops.prepare_binary_weights(w, 1, 1.0)
            return self.ops.binary_convolution_from_codes_prepared(codes, shape, self.prepared[name], None,
                                                                   (k // 2, k // 2), (stride, stride), (1, 1), DELTA)
        if name not in self.side:
            self.side[name] = (self.zeros_like(w), self.zeros_like(w, (w.shape[0],)))
        wb, alpha = self.side[name]
        return self.ops.binary_weight_convolution_from_codes(codes, shape, w, wb, alpha, None, (k // 2, k // 2),
                                                             (stride, stride), (1, 1), 1, 1.0, DELTA)

    def act_codes(self, a, bn_a, b=None, bn_b=None, b_codes=None):
        return self.ops.bn_add_relu_fixed_point_codes(a, self.bn_params(bn_a), b, self.bn_params(bn_b) if bn_b else None,
                                                      b_codes, DELTA, 1e-5, True, True, 8, DELTA)

    def _call_codes(self, x):
        o = self.ops
        h = o.convolution(x, self.p["stem/conv/W"], None, 1, (3, 3), (2, 2), (1, 1), 1)
        hc, shape = o.max_pooling_codes(self.act_codes(h, "stem/bn"), tuple(h.shape), (3, 3), (2, 2), True, (1, 1))
        cin = 64
        for s, (c, stride) in enumerate(STAGES):
            for b in range(2):
                st = stride if b == 0 else 1
                name = "stage%d/block%d" % (s + 1, b)
                r = self.bwconv_codes(name + "/conv1", hc, shape, 3, st)
                out_shape = tuple(r.shape)
                r = self.bwconv_codes(name + "/conv2", self.act_codes(r, name + "/bn1"), out_shape, 3, 1)
                if st != 1 or cin != c:
                    sc = self.bwconv_codes(name + "/shortcut", hc, shape, 1, st)
                    hc = self.act_codes(r, name + "/bn2", sc, name + "/bn_s")
                else:
                    hc = self.act_codes(r, name + "/bn2", b_codes=hc)
                shape, cin = out_shape, c
        g = o.global_average_pooling(o.codes_nhwc_to_float(hc, shape, DELTA))
        return o.affine(g, self.p["head/W"], self.p["head/b"], 1)

    def __call__(self, x):
        if self.fused == "codes":
            return self._call_codes(x)
        o = self.ops
        h = o.convolution(x, self.p["stem/conv/W"], None, 1, (3, 3), (2, 2), (1, 1), 1)
        self._rec("stem/conv", "convolution", [x], h)
        h = self.fused_act("stem/act", h, "stem/bn") if self.fused else self.relu_q("stem", self.bn("stem/bn", h), to_convolution=False)
        h = self._rec("stem/pool", "max_pooling", [h], o.max_pooling(h, (3, 3), (2, 2), True, (1, 1)))
        cin = 64
        for s, (c, stride) in enumerate(STAGES):
            for b in range(2):
                st = stride if b == 0 else 1
                name = "stage%d/block%d" % (s + 1, b)
                r = self.bwconv(name + "/conv1", h, 3, st)
                if self.fused:
                    r = self.fused_act(name + "/act1", r, name + "/bn1")
                    r = self.bwconv(name + "/conv2", r, 3, 1)
                    if st != 1 or cin != c:
                        sc = self.bwconv(name + "/shortcut", h, 1, st)
                        h = self.fused_act(name + "/act2", r, name + "/bn2", sc, name + "/bn_s")
                    else:
                        h = self.fused_act(name + "/act2", r, name + "/bn2", h)
                    cin = c
                    continue
                r = self.relu_q(name + "/act1", self.bn(name + "/bn1", r))
                r = self.bn(name + "/bn2", self.bwconv(name + "/conv2", r, 3, 1))
                if st != 1 or cin != c:
                    sc = self.bn(name + "/bn_s", self.bwconv(name + "/shortcut", h, 1, st))
                else:
                    sc = h
                a = self._rec(name + "/add", "add2", [r, sc], o.add2(r, sc))
                h = self.relu_q(name + "/act2", a)
                cin = c
        g = self._rec("head/pool", "global_average_pooling", [h], o.global_average_pooling(h))
        y = o.affine(g, self.p["head/W"], self.p["head/b"], 1)
        return self._rec("head/affine", "affine", [g], y)


# ---------------------------------------------------------------------------
# The same network with BatchNormalization folded into the convolutions
# ---------------------------------------------------------------------------

def fold_batch_normalization(params, eps=1e-5):
    """Folding constants of every BatchNormalization of the network, computed on the host in
    float32 exactly as nnabla's BatchNormalizationFolding converter computes them
    (python/src/nnabla/experimental/graph_converters/batch_normalization_folding.py:176-191):
    c0 = gamma / sqrt(var + eps), c1 = beta - gamma * mean / sqrt(var + eps); a convolution
    followed by that BN becomes a convolution with weights c0 * w and bias c1.
    Returns {bn name: (c0, c1)} (numpy float32)."""
    out = {}
    for key in params:
        if not key.endswith("/gamma"):
            continue
        name = key[:-len("/gamma")]
        host = lambda a: np.asarray(a.detach().cpu().numpy() if hasattr(a, "detach") else a, np.float32)
        beta, gamma = host(params[name + "/beta"]), host(params[name + "/gamma"])
        mean, var = host(params[name + "/mean"]), host(params[name + "/var"])
        std = np.sqrt(var + np.float32(eps))
        out[name] = (gamma / std, beta - (gamma * mean) / std)
    return out


def folded_layers():
    """(convolution name, BN name, kernel, stride) of the network's binary-weight layers, in order,
    with the block structure: yields ("block", name, cin, c, stride, has_shortcut)."""
    cin = 64
    for s, (c, stride) in enumerate(STAGES):
        for b in range(2):
            st = stride if b == 0 else 1
            yield "stage%d/block%d" % (s + 1, b), cin, c, st, (st != 1 or cin != c)
            cin = c


def folded_reference(ops, params, x, binarize, trace=None):
    """The folded graph on a plain function namespace (fp32 NCHW arrays; the oracle's): every
    Convolution -> BatchNormalization pair is one Convolution with folded weights and bias, as the
    converter leaves it, followed by the graph's own Add2 / ReLU / FixedPointQuantize /
    MaxPooling functions. `binarize(w)` returns (sign(w), alpha) of a binary-weight layer, whose
    effective weights sign(w) * alpha are what gets folded. trace (optional list) receives
    (layer name, output of the layer's quantizer or, for a shortcut branch, of its convolution)."""
    fold = fold_batch_normalization(params)
    f32 = np.float32

    def conv(name, bn, h, k, stride, binary=True):
        w = np.asarray(params[name + "/W"], f32)
        if binary:
            wb, alpha = binarize(w)
            w = wb * alpha.reshape(-1, 1, 1, 1)
        c0, c1 = fold[bn]
        return ops.convolution(h, (c0.reshape(-1, 1, 1, 1) * w).astype(f32), c1.astype(f32), 1, (k // 2, k // 2),
                               (stride, stride), (1, 1), 1)

    def rec(name, y):
        if trace is not None:
            trace.append((name, y))
        return y
    q = lambda v: ops.fixed_point_quantize(ops.relu(v), True, 8, DELTA)
    h = rec("stem", q(conv("stem/conv", "stem/bn", x, 7, 2, binary=False)))
    h = rec("stem/pool", ops.max_pooling(h, (3, 3), (2, 2), True, (1, 1)))
    for name, cin, c, st, has_sc in folded_layers():
        r = rec(name + "/conv1", q(conv(name + "/conv1", name + "/bn1", h, 3, st)))
        r = conv(name + "/conv2", name + "/bn2", r, 3, 1)
        sc = rec(name + "/shortcut", conv(name + "/shortcut", name + "/bn_s", h, 1, st)) if has_sc else h
        h = rec(name + "/conv2", q(ops.add2(r, sc)))
    g = ops.global_average_pooling(h)
    return ops.affine(g, params["head/W"], params["head/b"], 1)


class FoldedRunner:
    """The folded graph on the GPU: one kernel per convolution, each with its folded scale and
    bias, the residual addition, ReLU and FixedPointQuantize in its epilogue, int8 channel-last
    codes between the layers (nnabla_b200.functions.convolution_codes_folded). Weights are
    binarised and the folding constants computed once, at construction (a graph conversion, as
    the reference's converter is). The logits follow the folded graph, not the unfolded one bit
    for bit: folding moves roundings, as it does in the reference."""

    def __init__(self, ops, params, trace=None):
        import torch
        self.ops, self.trace = ops, trace
        dev = params["stem/conv/W"].device
        up = lambda a: torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(dev)
        host = lambda a: a.detach().cpu().numpy()
        fold = fold_batch_normalization(params)
        c0, c1 = fold["stem/bn"]
        self.stem_w = up(c0.reshape(-1, 1, 1, 1) * host(params["stem/conv/W"]))
        self.stem_b = up(c1)
        self.layers = {}

        def add(conv, bn):
            prep = ops.prepare_binary_weights(params[conv + "/W"], 1, 1.0)
            k0, k1 = fold[bn]
            scale = (host(prep.alpha) * k0).astype(np.float32) * np.float32(DELTA)
            self.layers[conv] = (prep, up(scale), up(k1))
        for name, cin, c, st, has_sc in folded_layers():
            add(name + "/conv1", name + "/bn1")
            add(name + "/conv2", name + "/bn2")
            if has_sc:
                add(name + "/shortcut", name + "/bn_s")
        self.head = (params["head/W"], params["head/b"])

    def _rec(self, name, x, y, shape, **kw):
        if self.trace is not None:
            self.trace.append(dict(layer=name, input=x, output=y, shape=shape, **kw))

    def __call__(self, x):
        o = self.ops
        hc, shape = o.convolution_relu_fixed_point_codes(x, self.stem_w, self.stem_b, (3, 3), (2, 2), True, True, 8,
                                                         DELTA)
        self._rec("stem", x, hc, shape)
        pc, pshape = o.max_pooling_codes(hc, shape, (3, 3), (2, 2), True, (1, 1))
        self._rec("stem/pool", hc, pc, pshape, in_shape=shape)
        hc, shape = pc, pshape
        for name, cin, c, st, has_sc in folded_layers():
            p1, s1, b1 = self.layers[name + "/conv1"]
            r, rshape = o.convolution_codes_folded(hc, shape, p1, s1, b1, (1, 1), (st, st), (1, 1))
            self._rec(name + "/conv1", hc, r, rshape, in_shape=shape, stride=st, k=3)
            p2, s2, b2 = self.layers[name + "/conv2"]
            if has_sc:
                ps, ss, bs = self.layers[name + "/shortcut"]
                sc, _ = o.convolution_codes_folded(hc, shape, ps, ss, bs, (0, 0), (st, st), (1, 1), relu=False,
                                                   output="float")
                self._rec(name + "/shortcut", hc, sc, rshape, in_shape=shape, stride=st, k=1)
                out, _ = o.convolution_codes_folded(r, rshape, p2, s2, b2, (1, 1), (1, 1), (1, 1), residual=sc)
                self._rec(name + "/conv2", r, out, rshape, in_shape=rshape, stride=1, k=3, residual=sc)
            else:
                out, _ = o.convolution_codes_folded(r, rshape, p2, s2, b2, (1, 1), (1, 1), (1, 1), residual_codes=hc,
                                                    residual_delta=DELTA)
                self._rec(name + "/conv2", r, out, rshape, in_shape=rshape, stride=1, k=3, residual_codes=hc)
            hc, shape = out, rshape
        g = o.global_average_pooling_codes(hc, shape, DELTA)
        return o.affine(g, self.head[0], self.head[1], 1)


def conv_macs_per_image(height=224, width=224, num_classes=1000):
    """Multiply-accumulates of the convolutions and the affine per image,
    counted from the layer shapes."""
    def out(v, k, s, p):
        return (v + 2 * p - k) // s + 1
    h, w = out(height, 7, 2, 3), out(width, 7, 2, 3)
    macs = 64 * 3 * 49 * h * w
    h, w = (h + 1 - 2) // 2 + 1, (w + 1 - 2) // 2 + 1
    cin = 64
    for c, stride in STAGES:
        for b in range(2):
            st = stride if b == 0 else 1
            ho, wo = out(h, 3, st, 1), out(w, 3, st, 1)
            macs += c * cin * 9 * ho * wo + c * c * 9 * ho * wo
            if st != 1 or cin != c:
                macs += c * cin * ho * wo
            h, w, cin = ho, wo, c
    return macs + 512 * num_classes
