"""Function namespaces with the names and argument order of nnabla_b200.functions, backed by
the CPU checkers (numpy arrays), so that one network definition runs on the GPU and on the
checker alike.

TEST INFRASTRUCTURE ONLY (tests, the smoke check and the benchmark's CPU baseline).
The module-level functions use the C restatement (oracle/oracle_*.c); `reference()` returns the
same namespace backed by the reference's own compiled functions (oracle/_ref), where built."""
import types

import numpy as np

from oracle import oracle


def convolution(x, w, b=None, base_axis=1, pad=None, stride=None, dilation=None, group=1, channel_last=False):
    return oracle.convolution(x, w, b, pad or (0, 0), stride or (1, 1), dilation or (1, 1), group)


def batch_normalization(x, beta, gamma, mean, var, axes=(1,), decay_rate=0.9, eps=1e-5, batch_stat=True,
                        output_stat=False):
    assert not batch_stat
    return oracle.batch_norm_inference(x, beta, gamma, mean, var, eps)


def relu(x, inplace=False):
    return oracle.relu(x)


def add2(a, b, inplace=False):
    return oracle.add2(a, b)


def fixed_point_quantize(x, sign=True, n=8, delta=2 ** -4, quantize=True, ste_fine_grained=True):
    return oracle.fixed_point_quantize(x, sign, n, delta)


def max_pooling(x, kernel, stride=None, ignore_border=True, pad=None, channel_last=False):
    return oracle.max_pooling(x, kernel, stride or kernel, ignore_border, pad or (0, 0))


def global_average_pooling(x):
    return oracle.global_average_pooling(x)


def binary_weight_convolution(x, w, wb, alpha, b=None, base_axis=1, pad=None, stride=None, dilation=None, group=1,
                              quantize_zero_to=1.0, **kw):
    y, wb_o, al_o = oracle.binary_weight_convolution(x, w, b, pad or (0, 0), stride or (1, 1), dilation or (1, 1),
                                                     group, quantize_zero_to)
    wb[...] = wb_o
    alpha[...] = al_o
    return y


def affine(x, w, b=None, base_axis=1, **kw):
    return oracle.affine(x, w, b, base_axis)


def bn_add_relu_fixed_point(a, bn_a, b=None, bn_b=None, eps=1e-5, relu_on=True, quantize=True, sign=True, n=8,
                            delta=2 ** -4):
    """The unfused chain the fused function must reproduce bit for bit."""
    v = oracle.batch_norm_inference(a, bn_a[0], bn_a[1], bn_a[2], bn_a[3], eps)
    if b is not None:
        w = oracle.batch_norm_inference(b, bn_b[0], bn_b[1], bn_b[2], bn_b[3], eps) if bn_b is not None else b
        v = oracle.add2(v, w)
    if relu_on:
        v = oracle.relu(v)
    return oracle.fixed_point_quantize(v, sign, n, delta) if quantize else v


def reference():
    """The same namespace on the reference's own CPU functions (oracle/_ref/libnnabla_ref.so);
    only what a residual network built from these functions calls."""
    from oracle import ref
    ns = types.SimpleNamespace()
    ns.convolution = lambda x, w, b=None, base_axis=1, pad=None, stride=None, dilation=None, group=1, \
        channel_last=False: ref.convolution(x, w, b, base_axis, pad or (0, 0), stride or (1, 1), dilation or (1, 1),
                                            group)

    def bn(x, beta, gamma, mean, var, axes=(1,), decay_rate=0.9, eps=1e-5, batch_stat=True, output_stat=False):
        # the reference wants the statistics shaped like x with 1 everywhere but the axis (batch_normalization.cpp:60-90)
        sh = [1] * x.ndim
        sh[axes[0]] = x.shape[axes[0]]
        r = lambda a: np.asarray(a, np.float32).reshape(sh)
        return ref.batch_normalization(x, r(beta), r(gamma), r(mean), r(var), tuple(axes), decay_rate, eps, batch_stat)
    ns.batch_normalization = bn
    ns.relu = lambda x, inplace=False: ref.relu(x)
    ns.add2 = lambda a, b, inplace=False: ref.add2(a, b)
    ns.fixed_point_quantize = lambda x, sign=True, n=8, delta=2 ** -4, quantize=True, ste_fine_grained=True: \
        ref.fixed_point_quantize(x, sign, n, delta)
    ns.max_pooling = lambda x, kernel, stride=None, ignore_border=True, pad=None, channel_last=False: \
        ref.max_pooling(x, kernel, stride or kernel, ignore_border, pad or (0, 0))
    ns.global_average_pooling = lambda x: ref.global_average_pooling(x)

    def bwc(x, w, wb, alpha, b=None, base_axis=1, pad=None, stride=None, dilation=None, group=1,
            quantize_zero_to=1.0, **kw):
        y, wb_o, al_o = ref.binary_weight_convolution(x, w, b, base_axis, pad or (0, 0), stride or (1, 1),
                                                      dilation or (1, 1), group, quantize_zero_to)
        wb[...] = wb_o
        alpha[...] = al_o
        return y
    ns.binary_weight_convolution = bwc
    ns.affine = lambda x, w, b=None, base_axis=1, **kw: ref.affine(x, w, b, base_axis)
    return ns


def binarize(w):
    """(sign(w), alpha) of a binary-weight convolution's weights [outmaps, ...]
    (binary_weight_convolution.cpp:81-104), for graphs that fold them into a plain convolution."""
    w = np.asarray(w, np.float32)
    wb, alpha, _ = oracle.binarize_rows(w.reshape(w.shape[0], -1), 1.0)
    return wb.reshape(w.shape), alpha
