#!/usr/bin/env python
"""Benchmark of the quantized-layer hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

Headline workload (BASELINE.json configs[1], the configuration the quantizer
GB/s metric is quoted on): one step = FixedPointQuantize(sign, n=8, delta=2^-4),
Pow2Quantize(sign, with_zero, n=8, m=1) and MinMaxQuantize(ql 0..255, given
per-tensor range -4..4) each applied to an fp32 tensor of 2^30 elements
~U(-4,4). Algorithmic traffic is 8 bytes per element per quantizer.

Prints ONE JSON line (rank 0). With N > 1 (torchrun) every rank processes its
own tensor: the path shards by elements with no collective (weak scaling).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BYTES_PER_ELEM = 8  # 4 read + 4 written, per quantizer
QUANTIZERS = ("fixed_point_quantize", "pow2_quantize", "min_max_quantize")
CPU_SAMPLE_LOG2 = 24


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--size-log2", type=int, default=30)
    ap.add_argument("--e2e-steps", type=int, default=2)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (profiling runs)")
    ap.add_argument("--no-extras", action="store_true", help="skip the other BASELINE configurations")
    ap.add_argument("--resnet-batch", type=int, default=256, help="images per GPU for the ResNet-18 extra")
    ap.add_argument("--only-extras", action="store_true",
                    help="run only the other BASELINE configurations and print their JSON (profiling runs)")
    ap.add_argument("--small-extras", action="store_true",
                    help="reduced sizes for the other configurations (ncu captures must stay small)")
    ap.add_argument("--backward-log2", type=int, default=0,
                    help="log2 of the element count of the quantizer-backward entry (default 28, 22 with --small-extras)")
    return ap.parse_args()


# --------------------------------------------------------------------------- CPU arm
def cpu_functions():
    """(kind, {name: callable(x)->seconds}) — the reference's own compiled CPU
    functions when oracle/_ref is present, else the C restatement."""
    from oracle import ref
    if ref.available():
        one = lambda v: np.array([v], np.float32)
        return "reference", {
            "fixed_point_quantize": lambda x: ref.fixed_point_quantize(x, True, 8, 2.0 ** -4, timed=True)[1],
            "pow2_quantize": lambda x: ref.pow2_quantize(x, True, True, 8, 1, timed=True)[1],
            "min_max_quantize": lambda x: ref.min_max_quantize(x, one(-4), one(4), one(0), one(255), timed=True)[3],
        }
    from oracle import oracle

    def timed(fn):
        def run(x):
            t0 = time.perf_counter()
            fn(x)
            return time.perf_counter() - t0
        return run
    return "port", {
        "fixed_point_quantize": timed(lambda x: oracle.fixed_point_quantize(x, True, 8, 2.0 ** -4)),
        "pow2_quantize": timed(lambda x: oracle.pow2_quantize(x, True, True, 8, 1)),
        "min_max_quantize": timed(lambda x: oracle.min_max_quantize(x, [-4], [4], [0], [255])),
    }


def cpu_step(fns, slices):
    """One bounded CPU step: every quantizer over every slice, one host thread
    per slice (the reference functions are single-threaded; independent
    function instances may run on separate threads). Returns wall seconds."""
    def work(x):
        for name in QUANTIZERS:
            fns[name](x)
    t0 = time.perf_counter()
    ths = [threading.Thread(target=work, args=(s,)) for s in slices]
    for t in ths:
        t.start()
    for t in ths:
        t.join()
    return time.perf_counter() - t0


def cpu_inputs(threads):
    rng = np.random.RandomState(0)
    n = 1 << CPU_SAMPLE_LOG2
    x = rng.uniform(-4, 4, n).astype(np.float32)
    per = n // threads
    return [x[i * per:(i + 1) * per] for i in range(threads)], per * threads


def cpu_contraction_samples():
    """CPU times of the GEMM / convolution configurations on bounded samples, beside the GPU
    numbers of `other_configs`. The reference multiplies through Eigen, which its build downloads
    and which is not in its tree; the contraction is therefore timed with the host's BLAS (NumPy)
    under the reference's control flow (sign / alpha passes, one unfold + one GEMM per sample,
    src/nbla/function/generic/convolution.cpp:160-197), once on 1 thread (the reference's CPU
    build is single-threaded) and once on all cores."""
    try:
        from threadpoolctl import threadpool_limits
    except ImportError:  # pragma: no cover - optional
        return {"unavailable": "threadpoolctl is missing"}
    rng = np.random.RandomState(0)
    f32 = np.float32
    out = {"blas": "NumPy's BLAS in place of Eigen (not vendored in the reference)"}

    def best_ms(fn, reps=2):
        ts = []
        for _ in range(reps):
            t0 = time.perf_counter()
            fn()
            ts.append(time.perf_counter() - t0)
        return 1e3 * min(ts)
    x0, w0 = rng.randn(256, 1024).astype(f32), (0.02 * rng.randn(1024, 4096)).astype(f32)

    def bwa():
        alpha = np.abs(w0).sum(0) * f32(1.0 / 1024)
        return x0 @ (np.where(w0 > 0, f32(1), f32(-1)) * alpha)
    rows = 512  # of 8192
    x2 = (np.rint(rng.randn(rows, 4096) * 32).clip(-127, 127) * f32(2.0 ** -5)).astype(f32)
    w2 = (np.rint(rng.randn(4096, 8192) * 20).clip(-127, 127) * f32(2.0 ** -10)).astype(f32)
    imgs = 4  # of 128
    x3 = np.maximum(rng.randn(imgs, 256, 28, 28), 0).astype(f32)
    w3 = (rng.randn(256, 2304) * np.sqrt(2.0 / 2304)).astype(f32)

    def bwc():
        alpha = np.abs(w3).sum(1) * f32(1.0 / 2304)
        wb = np.where(w3 > 0, f32(1), f32(-1)) * alpha[:, None]
        for i in range(imgs):
            xp = np.pad(x3[i], ((0, 0), (1, 1), (1, 1)))
            col = np.lib.stride_tricks.sliding_window_view(xp, (3, 3), axis=(1, 2))  # [256, 28, 28, 3, 3]
            col = np.ascontiguousarray(col.transpose(0, 3, 4, 1, 2)).reshape(2304, 784)
            wb @ col
    for label, threads in (("1_thread", 1), ("all_cores", os.cpu_count() or 1)):
        with threadpool_limits(limits=threads):
            out[label] = {
                "threads": threads,
                "configs[0] binary_weight_affine 256x1024x4096 ms": best_ms(bwa),
                "configs[2] affine 8192x4096x8192 ms (512 of 8192 rows timed, scaled x16)": 16 * best_ms(lambda: x2 @ w2),
                "configs[3] binary_weight_convolution batch 128 ms (4 images timed, scaled x32)": 32 * best_ms(bwc),
            }
    return out


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    kind, fns = cpu_functions()
    threads = os.cpu_count() or 1
    slices, n = cpu_inputs(threads)
    for _ in range(max(1, min(args.warmup, 1))):
        cpu_step(fns, slices)
    times = [cpu_step(fns, slices) for _ in range(args.steps)]
    total = sum(times)
    value = len(QUANTIZERS) * BYTES_PER_ELEM * n * args.steps / total / 1e9
    sample = "each step: 3 quantizers over 2^%d elements split over %d host threads" % (CPU_SAMPLE_LOG2, threads)
    line = {
        "impl": "reference", "metric": "quantizer_GBps", "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "configs[1]: FixedPoint+Pow2+MinMax quantize, fp32 U(-4,4); CPU arm on a bounded "
                               "sample of 2^%d elements per step" % CPU_SAMPLE_LOG2},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------- GPU arm
class ClockSampler:
    """Samples the SM clock and the clock-event (throttle) reasons of one GPU
    through NVML from a background thread while the timed region runs.
    Read-only: nothing about the GPU's settings is changed."""
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}

    def __init__(self, cuda_index, period_s=0.002):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        self.error = None
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            props = torch.cuda.get_device_properties(cuda_index)
            bus_id = "%08x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByPciBusId(bus_id.encode())
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception as exc:  # NVML missing: report it, do not fake clocks
            self.error = "%s: %s" % (type(exc).__name__, exc)
            return
        self._period = period_s
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                try:
                    bits = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                except AttributeError:
                    bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for bit, name in self.REASONS.items():
                    if bits & bit:
                        self.reasons.add(name)
            except Exception as exc:
                self.error = "%s: %s" % (type(exc).__name__, exc)
                return
            time.sleep(self._period)

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        out = {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
               "samples": len(self.samples), "reasons": sorted(self.reasons)}
        if self.error:
            out["error"] = self.error
        return out


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f), "measured"
    except OSError:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def time_gpu(fn, iters, warm=3):
    """Mean milliseconds per call of fn, CUDA events on the current stream."""
    import torch
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def run_extras(args, rank, world, barrier):
    """The other BASELINE configurations, timed per rank (inputs resident in
    HBM, tensors larger than L2 or an L2 flush between iterations is not
    applied to these short runs: stated per entry)."""
    import torch
    import torch.distributed as dist
    from nnabla_b200 import functions as F
    from nnabla_b200 import resnet18, sharding
    peaks, _ = measured_peaks()
    out = {}
    gen = torch.Generator(device="cuda").manual_seed(99 + rank)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=gen)

    def maxr(ms):
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return ms

    # configs[0]: BinaryWeightAffine 256 x 1024 x 4096 (replicated on every rank)
    M, K, N = 256, 1024, 4096
    x, w, b = rn(M, K), 0.02 * rn(K, N), torch.zeros(N, device="cuda")
    wb, al = torch.zeros_like(w), torch.zeros(N, device="cuda")
    ms = maxr(time_gpu(lambda: F.binary_weight_affine(x, w, wb, al, b), 50))
    out["configs[0] binary_weight_affine 256x1024x4096"] = {
        "ms": ms, "tflops_algorithmic": 2 * M * K * N / ms / 1e9, "tflops_issued_bf16x3": 6 * M * K * N / ms / 1e9,
        "frac_of_bf16_peak_issued": 6 * M * K * N / ms / 1e9 / peaks["bf16_tflops"],
        "includes": "binarise + alpha + split + GEMM, whole forward_impl", "l2": "working set fits L2 (latency-bound case)"}
    try:  # the same forward_impl recorded once as a CUDA graph: its five dependent launches replay as one
        from nnabla_b200 import graphs
        cap0 = graphs.Captured(lambda xx: F.binary_weight_affine(xx, w, wb, al, b), x)
        out["configs[0] binary_weight_affine 256x1024x4096"]["ms_cuda_graph"] = maxr(
            time_gpu(lambda: cap0.graph.replay(), 50))
        del cap0
    except RuntimeError as e:
        out["configs[0] binary_weight_affine 256x1024x4096"]["ms_cuda_graph"] = None
        out["configs[0] binary_weight_affine 256x1024x4096"]["cuda_graph_note"] = str(e)[:80]
    # configs[2]: 8-bit fixed-point affine, output columns sharded over the ranks
    M, K, N = (4096, 4096, 4096) if args.small_extras else (8192, 4096, 8192)
    Ns = N // world
    x = rn(M, K)
    w = 0.02 * rn(K, Ns)
    b = 0.01 * rn(Ns)
    xq, xc = F.fixed_point_quantize_with_codes(x, True, 8, 2.0 ** -5)
    wq, wc = F.fixed_point_quantize_with_codes(w, True, 8, 2.0 ** -10)
    ms_gemm = maxr(time_gpu(lambda: F.affine_from_codes(xc, wc, 2.0 ** -5, 2.0 ** -10, b), 20))
    wk = F.transpose_codes(wc)  # the weight's codes in the tensor core's layout, prepared once per weight update
    ms_prepared = maxr(time_gpu(lambda: F.affine_from_kmajor_codes(xc, wk, K, 2.0 ** -5, 2.0 ** -10, b), 20))
    entry = {"ms_gemm": ms_gemm, "int8_tops_whole_job": 2 * M * K * N / ms_gemm / 1e9,
             "ms_gemm_prepared_weights": ms_prepared,
             "int8_tops_whole_job_prepared_weights": 2 * M * K * N / ms_prepared / 1e9,
             "ms_gemm_includes": "ms_gemm re-lays the weight codes out K-major on every call (0.07 ms at the full "
                                 "size); ms_gemm_prepared_weights reuses a layout made once (transpose_codes)",
             "columns_per_gpu": Ns, "l2": "operands 32 MiB + 32 MiB/g int8; output 256 MiB/g fp32 exceeds L2"}
    ms_q = maxr(time_gpu(lambda: (F.fixed_point_quantize_with_codes(x, True, 8, 2.0 ** -5),
                                  F.fixed_point_quantize_with_codes(w, True, 8, 2.0 ** -10)), 10))
    entry["ms_quantize_x_and_w"] = ms_q
    try:  # the library's int8 GEMM on the same codes, for context only (int32 output, no scaling, no bias)
        wct = wc.t().contiguous().t()  # column-major B, the layout the library wants
        ms_lib = maxr(time_gpu(lambda: torch._int_mm(xc, wct), 20))
        entry["library_int8_gemm_ms"] = ms_lib
        entry["library_int8_tops_whole_job"] = 2 * M * K * N / ms_lib / 1e9
    except Exception as e:  # noqa: BLE001 - the comparison is optional
        entry["library_int8_gemm_ms"] = None
        entry["library_int8_note"] = str(e)[:100]
    if world > 1:
        def gemm_and_gather():
            yy = F.affine_from_codes(xc, wc, 2.0 ** -5, 2.0 ** -10, b)
            return sharding.gather_columns(yy, N)
        entry["ms_gemm_plus_allgather"] = maxr(time_gpu(gemm_and_gather, 10))
        entry["collective"] = "NCCL all-gather of the [8192, N/g] fp32 output slabs + interleave"
        # the same with the gather fused into the contraction: every rank's epilogue stores its slab into all
        # ranks' [M, N] results over NVLink (peer mappings), then one tiny all-reduce orders the ranks
        mats = sharding.PeerMatrices(M, N)

        def gemm_fused_gather():
            F.affine_from_codes_gather(xc, wc, 2.0 ** -5, 2.0 ** -10, b, mats.ptrs, rank, N, rank * Ns)
            mats.fence()
        entry["ms_gemm_fused_gather"] = maxr(time_gpu(gemm_fused_gather, 10))
        entry["fused_gather_equals_allgather"] = bool(torch.equal(mats.local, gemm_and_gather()))
        entry["fused_gather_GBps_out_per_gpu"] = (world - 1) * M * Ns * 4 / entry["ms_gemm_fused_gather"] / 1e6
        mats.close()
    out["configs[2] fixed-point int8 affine %dx%dx%d" % (M, K, N)] = entry
    del x, w, xq, wq, xc, wc
    # quantizer backward passes (straight-through estimators) on the configs[1] parameters, per rank
    nb = 1 << (args.backward_log2 or (22 if args.small_extras else 28))
    gx = torch.rand(nb, device="cuda", generator=gen) * 9 - 4.5
    gdy = rn(nb)
    gdx = torch.empty_like(gx)
    one = lambda v: torch.tensor([v], device="cuda")
    qa, qb, la, lb = one(-4.0), one(4.0), one(0.0), one(255.0)
    F.min_max_quantize(gx, qa, qb, la, lb)
    bw = {}
    for name, fn, bpe in (
            ("fixed_point", lambda: F.fixed_point_quantize_backward(gx, gdy, True, 8, 2.0 ** -4, True, False, gdx), 12),
            ("pow2", lambda: F.pow2_quantize_backward(gx, gdy, True, True, 8, 1, True, False, gdx), 12),
            ("min_max_dx_and_ranges", lambda: F.min_max_quantize_backward(gx, qa, qb, la, lb, gdy, grads=(gdx, None, None)), 12),
            ("fixed_point_accum", lambda: F.fixed_point_quantize_backward(gx, gdy, True, 8, 2.0 ** -4, True, True, gdx), 16),
            ("coarse_ste_copy", lambda: F.fixed_point_quantize_backward(gx, gdy, True, 8, 2.0 ** -4, False, False, gdx), 8)):
        ms = maxr(time_gpu(fn, 10))
        bw[name] = {"ms": ms, "GBps_per_gpu": bpe * nb / ms / 1e6, "bytes_per_element": bpe,
                    "frac_of_hbm_peak": bpe * nb / ms / 1e6 / peaks["hbm_gbs"]}
    out["quantizer backward, 2^%d elements per GPU" % (nb.bit_length() - 1)] = bw
    del gx, gdy, gdx
    # configs[3]: BinaryWeightConvolution 3x3, 256 -> 256, 28 x 28, batch 128 sharded over the ranks
    Nb = max(1, (16 if args.small_extras else 128) // world)
    x = torch.relu(rn(Nb, 256, 28, 28))
    w = rn(256, 256, 3, 3) * (2.0 / 2304) ** 0.5
    wb, al, b = torch.zeros_like(w), torch.zeros(256, device="cuda"), torch.zeros(256, device="cuda")
    ms = maxr(time_gpu(lambda: F.binary_weight_convolution(x, w, wb, al, b, 1, (1, 1), (1, 1)), 10))
    flops = 2.0 * (Nb * world * 28 * 28) * 256 * 2304
    out["configs[3] binary_weight_convolution 3x3 256->256 28x28 batch %d" % (Nb * world)] = {
        "ms": ms, "tflops_algorithmic_whole_job": flops / ms / 1e9, "tflops_issued_bf16x3_whole_job": 3 * flops / ms / 1e9,
        "frac_of_bf16_peak_issued_per_gpu": 3 * flops / world / ms / 1e9 / peaks["bf16_tflops"],
        "includes": "binarise + NCHW->NHWC split + implicit GEMM, whole forward_impl", "images_per_gpu": Nb}
    # backward of the same layer (straight-through weight gradient), per rank
    dyc = rn(Nb, 256, 28, 28)
    gxc, gwc, gbc = torch.empty_like(x), torch.empty_like(w), torch.empty(256, device="cuda")
    ms_dx = maxr(time_gpu(lambda: F.binary_weight_convolution_backward(
        x, wb, al, dyc, 1, (1, 1), (1, 1), propagate_down=(True, False, False), grads=(gxc, None, None)), 10))
    ms_dw = maxr(time_gpu(lambda: F.binary_weight_convolution_backward(
        x, wb, al, dyc, 1, (1, 1), (1, 1), propagate_down=(False, True, True), grads=(None, gwc, gbc)), 10))
    out["configs[3] backward (dx | dw + db), batch %d" % (Nb * world)] = {
        "ms_dx": ms_dx, "ms_dw_db": ms_dw, "tflops_algorithmic_dx_whole_job": flops / ms_dx / 1e9,
        "tflops_algorithmic_dw_whole_job": flops / ms_dw / 1e9,
        "includes": "operand re-layout (stuffing / batch-innermost transposes, bf16 pieces) + implicit GEMM"}
    del x, w, dyc, gxc
    # data-parallel gradient all-reduce of the ResNet-18 parameter set through the communicator (N > 1 only)
    if world > 1:
        from nnabla_b200 import communicators
        comm = communicators.MultiProcessDataParallelCommunicator()
        comm.init()
        shapes = [tuple(v.shape) for v in resnet18.init_parameters(np.random.RandomState(0)).values()]
        grads = [torch.ones(sh, device="cuda") for sh in shapes]
        n_par = sum(g.numel() for g in grads)
        cb = comm.all_reduce_callback(grads, pack_size=8 << 20, division=True)
        ms_ar = maxr(time_gpu(cb, 10))
        out["gradient all-reduce, ResNet-18 parameters"] = {
            "ms": ms_ar, "parameters": n_par, "arrays": len(grads), "bucket_values": 8 << 20,
            "bus_GBps": 2 * (world - 1) / world * n_par * 4 / ms_ar / 1e6,
            "correct": bool(all(torch.allclose(g, torch.ones_like(g)) for g in grads))}
    # configs[4]: binary-weight ResNet-18, batch sharded over the ranks
    B = args.resnet_batch
    Bg = max(1, B // world)
    params = {k: torch.from_numpy(v).cuda() for k, v in resnet18.init_parameters(np.random.RandomState(0)).items()}
    x = rn(Bg, 3, 224, 224)
    gz = lambda t, shape=None: torch.zeros(shape or tuple(t.shape), device="cuda")
    net = resnet18.Runner(F, params, gz)
    ms = maxr(time_gpu(lambda: net(x), 5, warm=2))
    F.check_device_status()
    net_fused = resnet18.Runner(F, params, gz, fused=True)
    ms_fused = maxr(time_gpu(lambda: net_fused(x), 5, warm=2))
    F.check_device_status()
    net_codes = resnet18.Runner(F, params, gz, fused="codes")
    ms_codes = maxr(time_gpu(lambda: net_codes(x), 5, warm=2))
    F.check_device_status()
    same = bool(torch.equal(net_codes(x), net(x)))
    net_prep = resnet18.Runner(F, params, gz, fused="codes", prepared_weights=True)
    ms_prep = maxr(time_gpu(lambda: net_prep(x), 5, warm=2))
    F.check_device_status()
    same = same and bool(torch.equal(net_prep(x), net(x)))
    # the same forward captured once as a CUDA graph and replayed (one launch instead of about 130 calls)
    from nnabla_b200 import graphs
    graph_note = "the int8-activations forward with prepared weights, captured once and replayed"
    try:
        captured = graphs.Captured(net_prep, x)
        ms_graph = time_gpu(lambda: captured(x), 5, warm=2)
        same = same and bool(torch.equal(captured(x), net(x)))
    except RuntimeError as e:  # a capture that another thread's CUDA call interrupted: report, do not fail the run
        ms_graph, graph_note = ms_prep, "capture failed (%s): eager time reported" % str(e)[:80]
    ms_graph = maxr(ms_graph)
    F.check_device_status()
    out["configs[4] binary-weight ResNet-18 224x224"] = {
        "ms_per_batch": ms, "images_per_sec_whole_job": Bg * world / ms * 1e3, "batch_per_gpu": Bg,
        "gmac_per_image": resnet18.conv_macs_per_image() / 1e9,
        "ms_per_batch_fused_activations": ms_fused,
        "images_per_sec_whole_job_fused_activations": Bg * world / ms_fused * 1e3,
        "fused": "BN (+ residual) + ReLU + FixedPointQuantize as one pass, bit-identical logits",
        "ms_per_batch_int8_activations": ms_codes,
        "images_per_sec_whole_job_int8_activations": Bg * world / ms_codes * 1e3,
        "int8_activations": "the fused pass writes int8 channel-last codes that the next convolution reads directly "
                            "(1 byte per activation between layers, residual = code * delta)",
        "ms_per_batch_int8_activations_prepared_weights": ms_prep,
        "images_per_sec_whole_job_int8_activations_prepared_weights": Bg * world / ms_prep * 1e3,
        "ms_per_batch_cuda_graph": ms_graph,
        "images_per_sec_whole_job_cuda_graph": Bg * world / ms_graph * 1e3,
        "cuda_graph": graph_note,
        "prepared_weights": "weights binarised once (inference: they do not change between calls) instead of in "
                            "every forward pass as the reference's forward_impl does",
        "int8_activations_logits_equal_unfused": same}
    return out


def run_b200_arm(args):
    import torch
    import torch.distributed as dist
    from nnabla_b200 import _capi as C
    from nnabla_b200 import functions as F

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    C.call("nb200_check_device")
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.only_extras:
        extras = run_extras(args, rank, world, barrier)
        if rank == 0:
            print(json.dumps({"other_configs": extras}))
        if world > 1:
            dist.destroy_process_group()
        return

    n = 1 << args.size_log2
    gen = torch.Generator(device="cuda").manual_seed(1234 + rank)
    x = torch.rand(n, device="cuda", generator=gen) * 8 - 4
    y = torch.empty_like(x)
    one = lambda v: torch.tensor([v], device="cuda", dtype=torch.float32)
    qr_min, qr_max, ql_min, ql_max = one(-4.0), one(4.0), one(0.0), one(255.0)

    def step(events=None):
        if events:
            events[0].record()
        F.fixed_point_quantize(x, True, 8, 2.0 ** -4, outputs=[y])
        if events:
            events[1].record()
        F.pow2_quantize(x, True, True, 8, 1, outputs=[y])
        if events:
            events[2].record()
        F.min_max_quantize(x, qr_min, qr_max, ql_min, ql_max, outputs=[y])
        if events:
            events[3].record()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(args.steps)]
    sampler = ClockSampler(local) if rank == 0 else None
    barrier()
    t_start = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)
    t_start.record()
    for s in range(args.steps):
        step(ev[s])
    t_end.record()
    barrier()
    clocks = sampler.stop() if sampler else None
    elapsed_ms = t_start.elapsed_time(t_end)
    if world > 1:
        t = torch.tensor([elapsed_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    per_kernel_ms = [statistics.mean(ev[s][k].elapsed_time(ev[s][k + 1]) for s in range(args.steps))
                     for k in range(3)]

    # ---- end to end through the host-buffer entry points -------------------
    e2e = None
    try:
        if args.no_e2e:
            raise RuntimeError("skipped by --no-e2e")
        hx = torch.empty(n, dtype=torch.float32, pin_memory=True)
        hy = torch.empty(n, dtype=torch.float32, pin_memory=True)
        hx.copy_(x)
        hq = np.array([-4.0, 4.0, 0.0, 255.0], np.float32)

        def e2e_step():
            C.call("nb200_fixed_point_quantize_f32_host", C.ptr(hx), C.ptr(hy), C.size_t(n), 1, 8,
                   C.c_float(2.0 ** -4))
            C.call("nb200_pow2_quantize_f32_host", C.ptr(hx), C.ptr(hy), C.size_t(n), 1, 1, 8, 1)
            C.call("nb200_min_max_quantize_f32_host", C.ptr(hx), C.size_t(n), C.ptr(hq[0:]), C.ptr(hq[1:]),
                   C.ptr(hq[2:]), C.ptr(hq[3:]), C.c_float(0.01), C.ptr(hy))

        e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            e2e_step()
        barrier()
        e2e_s = time.perf_counter() - t0
        if world > 1:
            t = torch.tensor([e2e_s], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_s = float(t.item())
        e2e = {"value": world * 3 * BYTES_PER_ELEM * n * args.e2e_steps / e2e_s / 1e9, "unit": "GB/s",
               "h2d_bytes_per_step": 3 * 4 * n, "d2h_bytes_per_step": 3 * 4 * n, "steps": args.e2e_steps,
               "api": "nb200_*_quantize_f32_host (pinned host buffers)"}
        del hx, hy
    except RuntimeError as exc:  # pinned allocation failure: report, do not fake
        e2e = {"value": None, "unit": "GB/s", "error": str(exc)[:200]}

    del x, y
    torch.cuda.empty_cache()
    extras = None
    if not args.no_extras:
        extras = run_extras(args, rank, world, barrier)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks, peak_kind = measured_peaks()
    value = world * 3 * BYTES_PER_ELEM * n * args.steps / (elapsed_ms / 1e3) / 1e9
    k_dom = int(np.argmax(per_kernel_ms))
    achieved = BYTES_PER_ELEM * n / (per_kernel_ms[k_dom] / 1e3) / 1e9
    # DRAM traffic per element of the dominant kernel from the committed ncu capture at 2^26 elements
    # (profiles/quantizers_2p26_full_capture.md), scaled to this launch: traffic grows with the element count.
    ncu_bytes_per_elem = {"fixed_point_quantize": 485.1e6 / 2 ** 26, "pow2_quantize": 485.4e6 / 2 ** 26,
                          "min_max_quantize": 486.9e6 / 2 ** 26}
    roofline = {"bound": "hbm", "kernel": QUANTIZERS[k_dom], "achieved": achieved, "peak": peaks["hbm_gbs"],
                "peak_source": peak_kind, "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                "traffic": ncu_bytes_per_elem[QUANTIZERS[k_dom]] * n, "traffic_unit": "bytes per launch",
                "algorithmic_bytes_per_launch": BYTES_PER_ELEM * n,
                "per_kernel_GBps": {QUANTIZERS[k]: BYTES_PER_ELEM * n / (per_kernel_ms[k] / 1e3) / 1e9
                                    for k in range(3)}}
    cpu_baseline = None
    if not args.no_cpu_baseline:
        kind, fns = cpu_functions()
        slices, ncpu = cpu_inputs(1)
        secs = {name: fns[name](slices[0]) for name in QUANTIZERS}
        cpu_baseline = {"value": 3 * BYTES_PER_ELEM * ncpu / sum(secs.values()) / 1e9, "unit": "GB/s", "cores": 1,
                        "kind": kind, "sample": "3 quantizers over 2^%d elements, 1 thread" % CPU_SAMPLE_LOG2,
                        "per_function_GBps": {k: BYTES_PER_ELEM * ncpu / v / 1e9 for k, v in secs.items()}}
        if not args.no_extras and rank == 0:
            cpu_baseline["other_configs"] = cpu_contraction_samples()
    line = {
        "metric": "quantizer_GBps", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "configs[1]: FixedPointQuantize(sign,n=8,delta=2^-4) + Pow2Quantize(sign,with_zero,"
                               "n=8,m=1) + MinMaxQuantize(0..255, range -4..4) on fp32 U(-4,4), 2^%d elements per GPU"
                               % args.size_log2,
                   "elements_per_gpu": n, "l2": "inputs (4 GiB) larger than L2; no flush needed"},
        "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "clocks": clocks,
        "gpu_launches": 4 * args.steps,
        "other_configs": extras,
    }
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_b200_arm(args)


if __name__ == "__main__":
    main()
