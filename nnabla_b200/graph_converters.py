"""Inference graph conversion for quantized networks: BatchNormalization folding plus fusion of each
layer's tail, in the manner of nnabla.experimental.graph_converters
(python/src/nnabla/experimental/graph_converters/batch_normalization_folding.py:92-200, which rewrites
Convolution -> BatchNormalization into one Convolution with W' = c0 * W, b' = c0 * b + c1).

nnabla's converters walk an nn.Variable graph. Here the graph is recorded from the network's own code:
the network is called once with a `Recorder` in place of the function namespace (nnabla.functions /
nnabla_b200.functions), which notes every call instead of computing it. `BatchNormalizationFolding.convert`
then matches, for every convolution,

    [BinaryWeight]Convolution -> BatchNormalization [-> Add2(., residual)] [-> ReLU] [-> FixedPointQuantize]

and emits one call per match: nnabla_b200.functions.convolution_codes_folded (int8 channel-last codes in and
out, folded scale and bias, residual, ReLU and quantizer in the kernel's epilogue) or, for a full-precision
first layer, convolution_relu_fixed_point_codes. MaxPooling and GlobalAveragePooling of quantized tensors
run on the codes. Anything else in the graph is refused (NotImplementedError): the converter never
falls back to another execution.

The folding constants are computed on the host in float32 exactly as the reference's converter does
(batch_normalization_folding.py:176-191): c0 = gamma / sqrt(var + eps), c1 = beta - gamma * mean / sqrt(var + eps).

`FusedBatchNormalization` (end of this file) is the milder conversion: only the activation tail
BatchNormalization [-> Add2] [-> ReLU] [-> FixedPointQuantize] becomes one function, everything keeps its
rounding and the result is the as-written graph's, bit for bit.
"""
import numpy as np


class Sym:
    """A tensor of the recorded graph."""

    def __init__(self, node=None):
        self.node = node          # producing Node (None: a graph input)
        self.consumers = []


class Node:
    def __init__(self, fn, inputs, attrs, index):
        self.fn, self.inputs, self.attrs, self.index = fn, inputs, attrs, index
        self.out = Sym(self)
        for s in inputs:
            if isinstance(s, Sym):
                s.consumers.append(self)


class Recorder:
    """Function namespace that records the calls of a network (the subset of nnabla.functions a
    quantized convolutional network is written with). Arrays passed as parameters are kept as they are."""

    def __init__(self):
        self.nodes = []
        self.input = Sym()

    def _add(self, fn, inputs, **attrs):
        n = Node(fn, inputs, attrs, len(self.nodes))
        self.nodes.append(n)
        return n.out

    def convolution(self, x, w, b=None, base_axis=1, pad=None, stride=None, dilation=None, group=1, **kw):
        return self._add("convolution", [x], w=w, b=b, pad=tuple(pad or (0, 0)), stride=tuple(stride or (1, 1)),
                         dilation=tuple(dilation or (1, 1)), group=group, base_axis=base_axis)

    def binary_weight_convolution(self, x, w, wb, alpha, b=None, base_axis=1, pad=None, stride=None, dilation=None,
                                  group=1, quantize_zero_to=1.0, **kw):
        return self._add("binary_weight_convolution", [x], w=w, b=b, pad=tuple(pad or (0, 0)),
                         stride=tuple(stride or (1, 1)), dilation=tuple(dilation or (1, 1)), group=group,
                         base_axis=base_axis, quantize_zero_to=quantize_zero_to)

    def batch_normalization(self, x, beta, gamma, mean, variance, axes=(1,), decay_rate=0.9, eps=1e-5,
                            batch_stat=True, output_stat=False):
        return self._add("batch_normalization", [x], beta=beta, gamma=gamma, mean=mean, var=variance,
                         axes=tuple(axes), eps=eps, batch_stat=batch_stat)

    def relu(self, x, inplace=False):
        return self._add("relu", [x])

    def add2(self, a, b, inplace=False):
        return self._add("add2", [a, b])

    def fixed_point_quantize(self, x, sign=True, n=8, delta=2 ** -4, quantize=True, ste_fine_grained=True):
        return self._add("fixed_point_quantize", [x], sign=sign, n=n, delta=delta)

    def max_pooling(self, x, kernel, stride=None, ignore_border=True, pad=None, channel_last=False):
        return self._add("max_pooling", [x], kernel=tuple(kernel), stride=tuple(stride or kernel),
                         ignore_border=ignore_border, pad=tuple(pad or (0, 0)))

    def global_average_pooling(self, x):
        return self._add("global_average_pooling", [x])

    def affine(self, x, w, b=None, base_axis=1, **kw):
        return self._add("affine", [x], w=w, b=b, base_axis=base_axis)


def _host(a):
    return np.asarray(a.detach().cpu().numpy() if hasattr(a, "detach") else a, np.float32)


def folding_constants(bn, eps=None):
    """(c0, c1) of a recorded BatchNormalization node, numpy float32, flat."""
    a = bn.attrs
    e = np.float32(a["eps"] if eps is None else eps)
    gamma = _host(a["gamma"]).reshape(-1) if a["gamma"] is not None else None
    beta = _host(a["beta"]).reshape(-1) if a["beta"] is not None else None
    mean, var = _host(a["mean"]).reshape(-1), _host(a["var"]).reshape(-1)
    std = np.sqrt(var + e)
    g = gamma if gamma is not None else np.ones_like(std)
    b = beta if beta is not None else np.zeros_like(std)
    return g / std, b - (g * mean) / std


class _Chain:
    """One convolution with the nodes folded into it."""

    def __init__(self, conv):
        self.conv, self.bn, self.add, self.relu, self.fxp = conv, None, None, None, None
        self.residual = None  # Sym added before the activation

    @property
    def last(self):
        for n in (self.fxp, self.relu, self.add, self.bn):
            if n is not None:
                return n
        return self.conv


def _single(sym, fn):
    """The only consumer of `sym` if it is a `fn` node, else None."""
    if len(sym.consumers) == 1 and sym.consumers[0].fn == fn:
        return sym.consumers[0]
    return None


class FoldedProgram:
    """The converted graph: a list of steps over an environment of run-time values."""

    def __init__(self, steps, input_sym, output_sym, calls):
        self.steps, self.input_sym, self.output_sym = steps, input_sym, output_sym
        self.calls = calls  # names of the library calls, in order (one per step)

    def __call__(self, x):
        env = {id(self.input_sym): x}
        for step in self.steps:
            step(env)
        return env[id(self.output_sym)]


class BatchNormalizationFolding:
    """convert(recorder, output_sym, ops) -> FoldedProgram running on `ops` (nnabla_b200.functions)."""

    def __init__(self, codes_bits=8):
        self.codes_bits = codes_bits

    def _chains(self, rec):
        chains, owner = [], {}
        for n in rec.nodes:
            if n.fn not in ("convolution", "binary_weight_convolution"):
                continue
            c = _Chain(n)
            c.bn = _single(n.out, "batch_normalization")
            if c.bn is not None:
                if c.bn.attrs["batch_stat"]:
                    raise NotImplementedError("BatchNormalization with batch_stat=True cannot be folded")
                if c.bn.attrs["axes"] != (1,):
                    raise NotImplementedError("only BatchNormalization over axis 1 is folded")
                tail = c.bn.out
                add = _single(tail, "add2")
                # the addition joins the chain that produces its FIRST operand; the second is the residual
                if add is not None and add.inputs[0] is tail:
                    c.add, c.residual, tail = add, add.inputs[1], add.out
                relu = _single(tail, "relu")
                if relu is not None:
                    c.relu, tail = relu, relu.out
                fxp = _single(tail, "fixed_point_quantize")
                if fxp is not None:
                    c.fxp = fxp
            for m in (c.conv, c.bn, c.add, c.relu, c.fxp):
                if m is not None:
                    owner[m.index] = c
            chains.append(c)
        return chains, owner

    def convert(self, rec, output_sym, ops):
        chains, owner = self._chains(rec)
        steps, calls = [], []
        kind = {id(rec.input): ("float",)}  # representation of every computed Sym: "float" (fp32 NCHW input),
        # "codes" (int8 channel-last + shape + delta), "nhwc" (fp32 channel-last residual), "plain" (fp32 result)

        def emit(name, fn):
            calls.append(name)
            steps.append(fn)

        def quant_of(c):
            a = c.fxp.attrs
            nn_ = a["n"] - 1 if a["sign"] else a["n"]
            if not (0 < nn_ <= 7):
                raise NotImplementedError("codes need n - sign <= 7 bits")
            return a["sign"], a["n"], float(a["delta"])

        done = set()
        # chains complete (and are emitted) at their last node; other nodes are emitted where they stand
        for n in rec.nodes:
            c = owner.get(n.index)
            if c is not None:
                if n is not c.last or id(c) in done:
                    continue
                done.add(id(c))
                self._emit_chain(c, kind, emit, ops, quant_of)
                continue
            src = n.inputs[0]
            k = kind.get(id(src))
            if n.fn == "max_pooling" and k is not None and k[0] == "codes":
                a = n.attrs

                def step(env, n=n, a=a, src=src):
                    codes, shape = env[id(src)]
                    env[id(n.out)] = ops.max_pooling_codes(codes, shape, a["kernel"], a["stride"], a["ignore_border"],
                                                          a["pad"])
                emit("max_pooling_codes", step)
                kind[id(n.out)] = k
            elif n.fn == "global_average_pooling" and k is not None and k[0] == "codes":
                def step(env, n=n, src=src, delta=k[1]):
                    codes, shape = env[id(src)]
                    env[id(n.out)] = ops.global_average_pooling_codes(codes, shape, delta)
                emit("global_average_pooling_codes", step)
                kind[id(n.out)] = ("plain",)
            elif n.fn == "affine" and k is not None and k[0] == "plain":
                def step(env, n=n, src=src):
                    env[id(n.out)] = ops.affine(env[id(src)], n.attrs["w"], n.attrs["b"], n.attrs["base_axis"])
                emit("affine", step)
                kind[id(n.out)] = ("plain",)
            else:
                raise NotImplementedError("%s of a %s tensor is not covered by the folded execution"
                                          % (n.fn, k[0] if k else "missing"))
        if id(output_sym) not in kind:
            raise NotImplementedError("the requested output is folded into another function")
        return FoldedProgram(steps, rec.input, output_sym, calls)

    def _emit_chain(self, c, kind, emit, ops, quant_of):
        import torch
        conv, a = c.conv, c.conv.attrs
        src = conv.inputs[0]
        k_in = kind.get(id(src))
        if k_in is None:
            raise NotImplementedError("a convolution's input is not available in the folded execution")
        if a["group"] != 1 or a["base_axis"] != 1:
            raise NotImplementedError("only group 1, base_axis 1 convolutions are folded")
        w = a["w"]
        dev = w.device
        to_dev = lambda arr: torch.from_numpy(np.ascontiguousarray(arr, np.float32)).to(dev)
        Ko = int(w.shape[0])
        c0, c1 = folding_constants(c.bn) if c.bn is not None else (np.ones(Ko, np.float32), np.zeros(Ko, np.float32))
        if a["b"] is not None:  # b' = c0 * b + c1
            c1 = c0 * _host(a["b"]).reshape(-1) + c1
        out = c.last.out
        if conv.fn == "convolution":
            # full-precision first layer: fp32 NCHW in, codes out
            if k_in[0] != "float" or c.add is not None or c.relu is None or c.fxp is None:
                raise NotImplementedError("a full-precision convolution is folded as Convolution -> BatchNormalization "
                                          "-> ReLU -> FixedPointQuantize of the network input")
            sign, n, delta = quant_of(c)
            wf, bf = to_dev(c0.reshape(-1, 1, 1, 1) * _host(w)), to_dev(c1)

            def step(env, src=src, out=out):
                env[id(out)] = ops.convolution_relu_fixed_point_codes(env[id(src)], wf, bf, a["pad"], a["stride"], True,
                                                                     sign, n, delta)
            emit("convolution_relu_fixed_point_codes", step)
            kind[id(out)] = ("codes", delta)
            return
        if k_in[0] != "codes":
            raise NotImplementedError("a binary-weight convolution is folded when its input is a quantized tensor")
        prep = ops.prepare_binary_weights(w, 1, a["quantize_zero_to"])
        scale = to_dev((_host(prep.alpha).reshape(-1) * c0).astype(np.float32) * np.float32(k_in[1]))
        bias = to_dev(c1)
        kw = {}
        res = c.residual
        if res is not None:
            k_res = kind.get(id(res))
            if k_res is None:
                raise NotImplementedError("the residual of an addition is not available in the folded execution")
        if c.fxp is not None:
            sign, n, delta = quant_of(c)
            if not sign:
                raise NotImplementedError("unsigned codes are not folded")
            kind[id(out)] = ("codes", delta)
            extra = dict(relu=c.relu is not None, n=n, delta=delta)
        else:
            if c.relu is not None or c.add is not None:
                raise NotImplementedError("a convolution tail without FixedPointQuantize is folded only as "
                                          "Convolution -> BatchNormalization")
            kind[id(out)] = ("nhwc",)
            extra = dict(relu=False, output="float")

        def step(env, src=src, out=out, res=res):
            codes, shape = env[id(src)]
            kw2 = dict(extra)
            if res is not None:
                if kind[id(res)][0] == "codes":
                    kw2["residual_codes"], kw2["residual_delta"] = env[id(res)][0], kind[id(res)][1]
                else:
                    kw2["residual"] = env[id(res)][0]
            env[id(out)] = ops.convolution_codes_folded(codes, shape, prep, scale, bias, a["pad"], a["stride"],
                                                        a["dilation"], **kw2)
        emit("convolution_codes_folded", step)


class FusedBatchNormalization:
    """The activation tail of every layer as ONE function, the other functions as they are:

        BatchNormalization [-> Add2(., BatchNormalization(s) | s)] [-> ReLU] [-> FixedPointQuantize]
            -> bn_add_relu_fixed_point(a, bn_a, b, bn_b, eps, relu, quantize, sign, n, delta)

    in the manner of nnabla's FusedBatchNormalization converter
    (python/src/nnabla/experimental/graph_converters/fused_batch_normalization.py, which rewrites
    BatchNormalization -> Add2 -> ReLU into the FusedBatchNormalization function); the quantizer that follows
    in a quantized network joins the same pass. Every operation keeps its own rounding, so the converted
    graph gives the as-written graph's result bit for bit, and each activation is read and written once
    instead of up to four times. A binary-weight convolution whose input comes out of a fused quantizer is
    told the quantizer's step (`fixed_point_delta`), which selects the exact int8 contraction.

    convert(recorder, output_sym, ops, zeros_like) -> FoldedProgram on `ops` (nnabla_b200.functions or a
    namespace of the same shape); zeros_like(w, shape=None) makes the Wb / alpha buffers of the binary layers."""

    class _Tail:
        def __init__(self, bn):
            self.bn, self.add, self.relu, self.fxp = bn, None, None, None
            self.other, self.other_bn = None, None  # second operand of the addition: Sym, and its BN node if any

        @property
        def last(self):
            for n in (self.fxp, self.relu, self.add):
                if n is not None:
                    return n
            return self.bn

    @staticmethod
    def _foldable(bn):
        return not bn.attrs["batch_stat"] and bn.attrs["axes"] == (1,)

    def _tails(self, rec):
        tails, owner = {}, {}  # by index of the tail's LAST node; node index -> tail
        for n in rec.nodes:
            if n.fn != "batch_normalization" or n.index in owner or not self._foldable(n):
                continue
            add = _single(n.out, "add2")
            if add is not None and add.inputs[1] is n.out and add.inputs[0] is not n.out:
                first = add.inputs[0].node
                if (first is not None and first.fn == "batch_normalization" and self._foldable(first)
                        and _single(first.out, "add2") is add):
                    continue  # the second operand's BN: taken in by the first operand's tail
            t = self._Tail(n)
            cur = n.out
            if add is not None and add.inputs[0] is not add.inputs[1]:
                t.add = add
                t.other = add.inputs[1] if add.inputs[0] is n.out else add.inputs[0]
                m = t.other.node
                if (m is not None and m.fn == "batch_normalization" and self._foldable(m)
                        and _single(m.out, "add2") is add and m.index not in owner
                        and float(m.attrs["eps"]) == float(n.attrs["eps"])):
                    t.other_bn = m
                cur = add.out
            relu = _single(cur, "relu")
            if relu is not None:
                t.relu, cur = relu, relu.out
            fxp = _single(cur, "fixed_point_quantize")
            if fxp is not None:
                t.fxp = fxp
            if t.last is t.bn:
                continue  # nothing to fuse with: stays a plain BatchNormalization
            for m in (t.bn, t.add, t.relu, t.fxp, t.other_bn):
                if m is not None:
                    owner[m.index] = t
            tails[t.last.index] = t
        return tails, owner

    def convert(self, rec, output_sym, ops, zeros_like):
        tails, owner = self._tails(rec)
        steps, calls = [], []
        step_of = {}  # Sym id -> quantizer step, for tensors that leave a fused quantizer
        side = {}

        def bn_tuple(node):
            a = node.attrs
            return (a["beta"], a["gamma"], a["mean"], a["var"])

        for n in rec.nodes:
            t = owner.get(n.index)
            if t is not None:
                if n is not t.last:
                    continue
                a_sym = t.bn.inputs[0]
                b_sym = None if t.add is None else (t.other_bn.inputs[0] if t.other_bn is not None else t.other)
                bn_a, bn_b = bn_tuple(t.bn), (bn_tuple(t.other_bn) if t.other_bn is not None else None)
                q = t.fxp.attrs if t.fxp is not None else dict(sign=True, n=8, delta=2 ** -4)
                args = (float(t.bn.attrs["eps"]), t.relu is not None, t.fxp is not None, q["sign"], q["n"], q["delta"])
                out = t.last.out
                if t.fxp is not None:
                    step_of[id(out)] = q["delta"]

                def step(env, a_sym=a_sym, b_sym=b_sym, bn_a=bn_a, bn_b=bn_b, args=args, out=out):
                    b = env[id(b_sym)] if b_sym is not None else None
                    env[id(out)] = ops.bn_add_relu_fixed_point(env[id(a_sym)], bn_a, b, bn_b, *args)
                steps.append(step)
                calls.append("bn_add_relu_fixed_point")
                continue
            a, src, out = n.attrs, n.inputs, n.out
            if n.fn == "fixed_point_quantize":
                step_of[id(out)] = a["delta"]
            if n.fn == "convolution":
                fn = lambda x, a=a: ops.convolution(x, a["w"], a["b"], a["base_axis"], a["pad"], a["stride"],
                                                    a["dilation"], a["group"])
            elif n.fn == "binary_weight_convolution":
                w = a["w"]
                side[n.index] = (zeros_like(w), zeros_like(w, (w.shape[0],)))
                hint = step_of.get(id(src[0]))
                kw = {"fixed_point_delta": hint} if hint is not None else {}
                fn = lambda x, a=a, s=side[n.index], kw=kw: ops.binary_weight_convolution(
                    x, a["w"], s[0], s[1], a["b"], a["base_axis"], a["pad"], a["stride"], a["dilation"], a["group"],
                    a["quantize_zero_to"], **kw)
            elif n.fn == "batch_normalization":
                fn = lambda x, a=a: ops.batch_normalization(x, a["beta"], a["gamma"], a["mean"], a["var"], list(a["axes"]),
                                                            0.9, a["eps"], a["batch_stat"])
            elif n.fn == "relu":
                fn = lambda x: ops.relu(x)
            elif n.fn == "add2":
                fn = lambda x, y: ops.add2(x, y)
            elif n.fn == "fixed_point_quantize":
                fn = lambda x, a=a: ops.fixed_point_quantize(x, a["sign"], a["n"], a["delta"])
            elif n.fn == "max_pooling":
                fn = lambda x, a=a: ops.max_pooling(x, a["kernel"], a["stride"], a["ignore_border"], a["pad"])
                if id(src[0]) in step_of:
                    step_of[id(out)] = step_of[id(src[0])]  # the maximum of multiples of a step is one of them
            elif n.fn == "global_average_pooling":
                fn = lambda x: ops.global_average_pooling(x)
            elif n.fn == "affine":
                fn = lambda x, a=a: ops.affine(x, a["w"], a["b"], a["base_axis"])
            else:
                raise NotImplementedError("no rule for the function %s" % n.fn)

            def step(env, fn=fn, src=src, out=out):
                env[id(out)] = fn(*[env[id(s)] for s in src])
            steps.append(step)
            calls.append(n.fn)
        return FoldedProgram(steps, rec.input, output_sym, calls)
