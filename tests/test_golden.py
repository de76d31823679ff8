"""The C restatement against the committed golden vectors (produced by the
reference's own CPU functions). Runs without the reference checkout."""
import numpy as np
import pytest

import cases
from golden_util import bits, golden, sha
from oracle import oracle


@pytest.mark.parametrize("i", range(len(cases.FXP_GRID)))
def test_fxp(i):
    g = golden()
    sign, n, delta = g[f"fxp{i}/args"]
    got = oracle.fixed_point_quantize(g[f"fxp{i}/x"], bool(sign), int(n), float(delta))
    assert np.array_equal(bits(got), bits(g[f"fxp{i}/out"]))


@pytest.mark.parametrize("i", range(len(cases.POW2_GRID) + 1))
def test_pow2(i):
    g = golden()
    sign, wz, n, m = g[f"pow2_{i}/args"]
    got = oracle.pow2_quantize(g["pow2/x"], bool(sign), bool(wz), int(n), int(m))
    assert np.array_equal(bits(got), bits(g[f"pow2_{i}/out"]))


@pytest.mark.parametrize("i", range(len(cases.MINMAX_GRID)))
def test_minmax(i):
    g = golden()
    decay, xmm, ema, eps = g[f"minmax{i}/args"]
    x, qmin, qmax, lmin, lmax = cases.minmax_inputs(tuple(g[f"minmax{i}/xshape"]), tuple(g[f"minmax{i}/qshape"]))
    y, amin, amax, _ = oracle.min_max_quantize(x, qmin, qmax, lmin, lmax, float(decay), bool(xmm), bool(ema), float(eps))
    assert np.array_equal(sha(y), g[f"minmax{i}/out_sha"])
    assert np.array_equal(bits(amin), bits(g[f"minmax{i}/out_qr_min"]))
    assert np.array_equal(bits(amax), bits(g[f"minmax{i}/out_qr_max"]))


@pytest.mark.parametrize("i", range(len(cases.AFFINE_CASES)))
@pytest.mark.parametrize("qzt", cases.QZT)
def test_binary_affine(i, qzt):
    g = golden()
    xs, ws, ba = cases.AFFINE_CASES[i]
    x, w, b = cases.affine_inputs(xs, ws, with_zeros=True)
    y, wb, al = oracle.binary_weight_affine(x, w, b, ba, qzt)
    k = f"bwa{i}_{int(qzt)}"
    assert np.array_equal(bits(wb), bits(g[k + "/out_wb"]))
    np.testing.assert_allclose(al, g[k + "/out_alpha"], rtol=1e-6)
    assert cases.rel_rms(y, g[k + "/out_y"]) < 1e-6
    y, wb = oracle.binary_connect_affine(x, w, b, ba, qzt)
    k = f"bca{i}_{int(qzt)}"
    assert np.array_equal(bits(wb), bits(g[k + "/out_wb"]))
    assert cases.rel_rms(y, g[k + "/out_y"]) < 1e-6


@pytest.mark.parametrize("i", range(len(cases.CONV_CASES)))
def test_binary_convolution(i):
    g = golden()
    xs, ws, pad, stride, dil, grp = cases.CONV_CASES[i]
    x, w, b = cases.conv_inputs(xs, ws, with_zeros=True)
    y, wb, al = oracle.binary_weight_convolution(x, w, b, pad, stride, dil, grp, 1.0)
    assert np.array_equal(bits(wb), bits(g[f"bwc{i}/out_wb"]))
    np.testing.assert_allclose(al, g[f"bwc{i}/out_alpha"], rtol=1e-6)
    assert cases.rel_rms(y, g[f"bwc{i}/out_y"]) < 1e-6
    y, wb = oracle.binary_connect_convolution(x, w, b, pad, stride, dil, grp, 1.0)
    assert np.array_equal(bits(wb), bits(g[f"bcc{i}/out_wb"]))
    assert cases.rel_rms(y, g[f"bcc{i}/out_y"]) < 1e-6


def test_baseline_config_digests():
    g = golden()
    rng = np.random.RandomState(0)
    x = rng.uniform(-4, 4, 1 << 20).astype(np.float32)
    one = lambda v: np.array([v], np.float32)
    assert np.array_equal(sha(oracle.fixed_point_quantize(x, True, 8, 2.0 ** -4)), g["cfg2_fxp/sha"])
    assert np.array_equal(sha(oracle.pow2_quantize(x, True, True, 8, 1)), g["cfg2_pow2/sha"])
    assert np.array_equal(sha(oracle.min_max_quantize(x, one(-4), one(4), one(0), one(255))[0]), g["cfg2_minmax/sha"])


# ---- quantizer backward passes against golden_backward.npz -----------------
import backward_cases  # noqa: E402


@pytest.mark.parametrize("i", range(len(cases.FXP_GRID)))
@pytest.mark.parametrize("fine,accum", backward_cases.FLAGS)
def test_fxp_backward(i, fine, accum):
    backward_cases.check_fxp(oracle, i, fine, accum)


@pytest.mark.parametrize("i", range(len(backward_cases.POW2_CASES)))
@pytest.mark.parametrize("fine,accum", backward_cases.FLAGS)
def test_pow2_backward(i, fine, accum):
    backward_cases.check_pow2(oracle, i, fine, accum)


@pytest.mark.parametrize("i", range(len(cases.MINMAX_GRID)))
@pytest.mark.parametrize("fine,accum", backward_cases.FLAGS)
def test_minmax_backward(i, fine, accum):
    backward_cases.check_minmax(oracle, i, fine, accum)


# ---- sibling quantization functions against golden_siblings.npz ------------
import sibling_cases  # noqa: E402


@pytest.mark.parametrize("name", ["binary_sigmoid", "binary_tanh"])
@pytest.mark.parametrize("accum", [False, True])
def test_sibling_binary(name, accum):
    sibling_cases.check_binary(oracle, name, accum)


@pytest.mark.parametrize("i", range(len(cases.QL_GRID)))
def test_sibling_quantize_linear(i):
    sibling_cases.check_quantize_linear(oracle, i)


@pytest.mark.parametrize("i", range(len(cases.QL_SHAPES)))
@pytest.mark.parametrize("accum", [False, True])
def test_sibling_linear_rest(i, accum):
    sibling_cases.check_linear_rest(oracle, i, accum)


# ---- training side of the companions against golden_companions.npz ----------

def _gc():
    import os
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_companions.npz"))


@pytest.mark.parametrize("i", range(3))
def test_companions_batch_normalization_training(i):
    import companion_cases as cc
    g, c = _gc(), cc.bn_case(i)
    got = oracle.batch_norm_batch(c["x"], c["beta"], c["gamma"], c["mean"], c["var"])
    for k, a in zip(("y", "m", "v", "rm", "rv"), got):
        assert np.array_equal(bits(a).reshape(-1), bits(g["bn%d/fwd_%s" % (i, k)]).reshape(-1)), k
    for batch_stat in (True, False):
        m, v = (got[1], got[2]) if batch_stat else (c["mean"], c["var"])
        for accum in (False, True):
            r = oracle.batch_norm_backward(c["x"], c["dy"], c["gamma"], m, v, 1e-5, batch_stat,
                                           c["dmean"] if batch_stat else None, c["dvar"] if batch_stat else None,
                                           accum=(accum,) * 3, grads=c["g0"])
            k = "bn%d/bwd_%d%d" % (i, int(batch_stat), int(accum))
            for a, nm in zip(r, ("dx", "dbeta", "dgamma")):
                assert np.array_equal(bits(a).reshape(-1), bits(g[k + "_" + nm]).reshape(-1)), (k, nm)


def test_companions_backward_elementwise_and_pooling():
    import companion_cases as cc
    g = _gc()
    for i in range(len(cc.POOL_CASES)):
        c = cc.pool_case(i)
        for accum in (False, True):
            got = oracle.max_pooling_backward(c["x"], g["pool%d/dy" % i], c["kernel"], c["stride"], c["ib"], c["pad"],
                                              accum, c["g0"])
            assert np.array_equal(bits(got), bits(g["pool%d/dx_%d" % (i, int(accum))]))
    e = cc.elementwise_case()
    for accum in (False, True):
        assert np.array_equal(bits(oracle.relu_backward(oracle.relu(e["x"]), e["dy"], accum, e["g0"])),
                              bits(g["relu/dx_%d" % accum]))
        assert np.array_equal(bits(oracle.add2_backward(e["dy"], accum, e["g0"])), bits(g["add2/dx_%d" % accum]))
        assert np.array_equal(bits(oracle.global_average_pooling_backward(e["x"].shape, e["dyp"], accum, e["g0"])),
                              bits(g["gap/dx_%d" % accum]))
