"""GPU parity of the affine layers (tcgen05 contractions) through the C ABI:
signs bit-exact, alpha to 1e-6, outputs within 1e-5 of the output RMS of the
oracle (1e-5 of the output RMS, the tolerance the benchmark definition states for GEMM outputs)."""
import numpy as np
import pytest
import torch

import cases
from golden_util import bits, golden, sha
from oracle import oracle

pytestmark = pytest.mark.gpu
TOL = 1e-5  # of output RMS


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).cuda()


@pytest.fixture(scope="module")
def F():
    from nnabla_b200 import _capi, functions
    _capi.call("nb200_check_device")
    return functions


def run_bwa(F, x, w, b, base_axis, qzt):
    wb = torch.zeros(w.shape, device="cuda")
    al = torch.zeros(int(np.prod(w.shape[1:])), device="cuda")
    y = F.binary_weight_affine(dev(x), dev(w), wb, al, dev(b) if b is not None else None, base_axis, qzt)
    F.check_device_status()
    return y.cpu().numpy(), wb.cpu().numpy(), al.cpu().numpy()


@pytest.mark.parametrize("i", range(len(cases.AFFINE_CASES)))
@pytest.mark.parametrize("qzt", cases.QZT)
def test_binary_affine_golden(F, i, qzt):
    g = golden()
    xs, ws, ba = cases.AFFINE_CASES[i]
    x, w, b = cases.affine_inputs(xs, ws, with_zeros=True)
    y, wb, al = run_bwa(F, x, w, b, ba, qzt)
    k = f"bwa{i}_{int(qzt)}"
    assert np.array_equal(bits(wb), bits(g[k + "/out_wb"]))
    np.testing.assert_allclose(al, g[k + "/out_alpha"], rtol=1e-6)
    assert y.shape == g[k + "/out_y"].shape
    assert cases.rel_rms(y, g[k + "/out_y"]) < TOL
    wbc = torch.zeros(w.shape, device="cuda")
    yc = F.binary_connect_affine(dev(x), dev(w), wbc, dev(b), ba, qzt)
    F.check_device_status()
    k = f"bca{i}_{int(qzt)}"
    assert np.array_equal(bits(wbc.cpu().numpy()), bits(g[k + "/out_wb"]))
    assert cases.rel_rms(yc.cpu().numpy(), g[k + "/out_y"]) < TOL


@pytest.mark.parametrize("M,K,N", [(1, 8, 16), (5, 64, 24), (129, 200, 130), (256, 1024, 512), (300, 72, 1000)])
@pytest.mark.parametrize("bias", [True, False])
def test_binary_weight_affine_shapes(F, M, K, N, bias):
    rng = np.random.RandomState(M + K + N)
    x = rng.randn(M, K).astype(np.float32)
    w = (0.02 * rng.randn(K, N)).astype(np.float32)
    b = rng.randn(N).astype(np.float32) if bias else None
    y, wb, al = run_bwa(F, x, w, b, 1, 1.0)
    wy, wwb, wal = oracle.binary_weight_affine(x, w, b, 1, 1.0)
    assert np.array_equal(bits(wb), bits(wwb))
    # alpha: the reference sums |w| with Eigen, the oracle sequentially in fp32
    # (rounding error grows with K); the GPU sums in a fixed blocked order.
    # Both must sit within fp32 summation error of the exact mean.
    exact = np.abs(w.astype(np.float64)).mean(0)
    np.testing.assert_allclose(al, exact, rtol=1e-6)
    np.testing.assert_allclose(al, wal, rtol=1e-6 + K * 6e-8)
    assert cases.rel_rms(y, wy) < TOL


def test_binary_weight_affine_config1(F):
    """BASELINE configs[0]: x [256,1024], W [1024,4096], bias zeros, quantize_zero_to = 1."""
    g = golden()
    rng = np.random.RandomState(0)
    x = rng.randn(256, 1024).astype(np.float32)
    w = (0.02 * rng.randn(1024, 4096)).astype(np.float32)
    y, wb, al = run_bwa(F, x, w, np.zeros(4096, np.float32), 1, 1.0)
    assert np.array_equal(sha(wb), g["cfg1/wb_sha"])
    np.testing.assert_allclose(al, np.abs(w.astype(np.float64)).mean(0), rtol=1e-6)
    np.testing.assert_allclose(al, g["cfg1/alpha"], rtol=1e-6 + 1024 * 6e-8)  # reference sum is sequential fp32
    rms = float(g["cfg1/y_rms"][0])
    err = np.sqrt(np.mean((y[:4].astype(np.float64) - g["cfg1/y_rows"]) ** 2))
    assert err / rms < TOL
    wy = oracle.affine(x, np.where(w > 0, 1, np.where(w < 0, -1, 1)).astype(np.float32) * al[None, :], None, 1, f64=True)
    print("config1 rel-RMS error vs fp64 product:", cases.rel_rms(y, wy))
    assert cases.rel_rms(y, wy) < TOL


def test_fixed_point_affine_is_exact(F):
    """BASELINE configs[2] at a reduced size: both operands 8-bit fixed point;
    the int8 path must reproduce the fp32 oracle bit for bit (every partial
    sum is an integer below 2^24 times a power of two)."""
    rng = np.random.RandomState(0)
    M, K, N = 384, 512, 640
    x = rng.randn(M, K).astype(np.float32)
    w = (0.02 * rng.randn(K, N)).astype(np.float32)
    b = (0.01 * rng.randn(N)).astype(np.float32)
    xq = F.fixed_point_quantize(dev(x), True, 8, 2.0 ** -5)
    wq = F.fixed_point_quantize(dev(w), True, 8, 2.0 ** -10)
    y = F.affine(xq, wq, dev(b), fixed_point=(2.0 ** -5, 2.0 ** -10))
    F.check_device_status()
    want = oracle.affine(oracle.fixed_point_quantize(x, True, 8, 2.0 ** -5),
                         oracle.fixed_point_quantize(w, True, 8, 2.0 ** -10), b)
    assert np.array_equal(bits(y.cpu().numpy()), bits(want))
    # the same through the codes the quantizer emits
    _, xc = F.fixed_point_quantize_with_codes(dev(x), True, 8, 2.0 ** -5)
    _, wc = F.fixed_point_quantize_with_codes(dev(w), True, 8, 2.0 ** -10)
    y2 = F.affine_from_codes(xc, wc, 2.0 ** -5, 2.0 ** -10, dev(b))
    F.check_device_status()
    assert np.array_equal(bits(y2.cpu().numpy()), bits(want))


@pytest.mark.parametrize("M,K,N", [(7, 33, 50), (128, 256, 1000), (260, 512, 96)])
def test_fixed_point_affine_ragged(F, M, K, N):
    rng = np.random.RandomState(K)
    xq = oracle.fixed_point_quantize(rng.randn(M, K).astype(np.float32), True, 8, 2.0 ** -5)
    wq = oracle.fixed_point_quantize((0.02 * rng.randn(K, N)).astype(np.float32), True, 8, 2.0 ** -10)
    y = F.affine(dev(xq), dev(wq), None, fixed_point=(2.0 ** -5, 2.0 ** -10))
    F.check_device_status()
    assert np.array_equal(bits(y.cpu().numpy()), bits(oracle.affine(xq, wq, None)))


@pytest.mark.parametrize("M,K,N", [(4, 512, 1000), (130, 100, 70)])
def test_full_precision_affine(F, M, K, N):
    rng = np.random.RandomState(N)
    x = rng.randn(M, K).astype(np.float32)
    w = rng.randn(K, N).astype(np.float32)
    b = rng.randn(N).astype(np.float32)
    y = F.affine(dev(x), dev(w), dev(b))
    F.check_device_status()
    assert cases.rel_rms(y.cpu().numpy(), oracle.affine(x, w, b, f64=True)) < TOL


def test_shape_errors(F):
    x = torch.zeros(4, 8, device="cuda")
    w = torch.zeros(9, 3, device="cuda")
    with pytest.raises(RuntimeError, match="mismatch"):
        F.binary_weight_affine(x, w, torch.zeros_like(w), torch.zeros(3, device="cuda"))
    w = torch.zeros(8, 3, device="cuda")
    with pytest.raises(RuntimeError, match="alpha"):
        F.binary_weight_affine(x, w, torch.zeros_like(w), torch.zeros(4, device="cuda"))
    with pytest.raises(RuntimeError, match="bf16"):
        F.binary_weight_affine(x, w, torch.zeros_like(w), torch.zeros(3, device="cuda"), quantize_zero_to=0.3)


@pytest.mark.parametrize("M,K,N", [(2304, 256, 2304), (2500, 200, 2400)])
def test_large_fixed_point_affine_two_sm_tiles(F, M, K, N):
    """Large enough for the two-SM (CTA pair) kernel, including ragged edges:
    exact against integer arithmetic done in float64."""
    rng = np.random.RandomState(M)
    xq = oracle.fixed_point_quantize(rng.randn(M, K).astype(np.float32), True, 8, 2.0 ** -5)
    wq = oracle.fixed_point_quantize((0.02 * rng.randn(K, N)).astype(np.float32), True, 8, 2.0 ** -10)
    b = (0.01 * rng.randn(N)).astype(np.float32)
    y = F.affine(dev(xq), dev(wq), dev(b), fixed_point=(2.0 ** -5, 2.0 ** -10))
    F.check_device_status()
    exact = (xq.astype(np.float64) @ wq.astype(np.float64)).astype(np.float32) + b  # the product is exact in fp32
    assert np.array_equal(bits(y.cpu().numpy()), bits(exact))


def test_large_binary_weight_affine_two_sm_tiles(F):
    rng = np.random.RandomState(5)
    M, K, N = 2304, 192, 2400
    x = rng.randn(M, K).astype(np.float32)
    w = (0.02 * rng.randn(K, N)).astype(np.float32)
    b = rng.randn(N).astype(np.float32)
    y, wb, al = run_bwa(F, x, w, b, 1, 1.0)
    sgn = np.where(w > 0, 1.0, np.where(w < 0, -1.0, 1.0))
    assert np.array_equal(wb, sgn.astype(np.float32))
    want = (x.astype(np.float64) @ sgn) * np.abs(w.astype(np.float64)).mean(0) + b
    assert cases.rel_rms(y, want) < TOL


@pytest.mark.parametrize("M,K,N", [(384, 512, 640), (70, 200, 333), (2304, 256, 2304)])
def test_affine_from_prepared_kmajor_codes(F, M, K, N):
    rng = np.random.RandomState(M + N)
    x = rng.randn(M, K).astype(np.float32)
    w = (0.02 * rng.randn(K, N)).astype(np.float32)
    b = (0.01 * rng.randn(N)).astype(np.float32)
    _, xc = F.fixed_point_quantize_with_codes(dev(x), True, 8, 2.0 ** -5)
    _, wc = F.fixed_point_quantize_with_codes(dev(w), True, 8, 2.0 ** -10)
    want = F.affine_from_codes(xc, wc, 2.0 ** -5, 2.0 ** -10, dev(b))
    wk = F.transpose_codes(wc)
    got = F.affine_from_kmajor_codes(xc, wk, K, 2.0 ** -5, 2.0 ** -10, dev(b))
    F.check_device_status()
    assert torch.equal(got, want)


def test_fixed_point_affine_full_baseline_size(F):
    """BASELINE configs[2] at its full size (8192 x 4096 x 8192): every partial sum is an
    integer below 2^24 times a power of two, so the result is exact and must equal, bit for
    bit, an independent integer product (the library's int8 GEMM, used here as a checker only)
    scaled and biased with one rounding each; a window of rows is also checked against the
    oracle."""
    M, K, N = 8192, 4096, 8192
    gen = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(M, K, device="cuda", generator=gen)
    w = 0.02 * torch.randn(K, N, device="cuda", generator=gen)
    b = 0.01 * torch.randn(N, device="cuda", generator=gen)
    xq, xc = F.fixed_point_quantize_with_codes(x, True, 8, 2.0 ** -5)
    wq, wc = F.fixed_point_quantize_with_codes(w, True, 8, 2.0 ** -10)
    y = F.affine_from_codes(xc, wc, 2.0 ** -5, 2.0 ** -10, b)
    y2 = F.affine_from_kmajor_codes(xc, F.transpose_codes(wc), K, 2.0 ** -5, 2.0 ** -10, b)
    F.check_device_status()
    assert torch.equal(y, y2)
    acc = torch._int_mm(xc, wc.t().contiguous().t())
    want = acc.float().mul_(2.0 ** -15).add_(b)
    assert torch.equal(y, want)
    rows = slice(4000, 4016)
    ref_rows = oracle.affine(xq[rows].cpu().numpy(), wq.cpu().numpy(), b.cpu().numpy())
    assert np.array_equal(bits(y[rows].cpu().numpy()), bits(ref_rows))
