#!/usr/bin/env python
"""Benchmark of the quantized-layer hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

Headline workload: the binary-weight ResNet-18 (first convolution and final
affine full precision, every other convolution a BinaryWeightConvolution,
FixedPointQuantize(n=8, delta=2^-4) after each ReLU, BatchNormalization on
running statistics), random initialisation, input fp32 [256, 3, 224, 224]
~N(0,1), 1000 classes. One step = one forward pass of the whole batch; with N
GPUs (torchrun, one process per GPU) the batch is sharded, 256 / N images per
GPU, weights replicated, no collective in the forward pass (strong scaling).
`value` is images per second of the graph AS IT IS WRITTEN, function by
function through nnabla_b200.functions; the other execution forms of the same
graph (fused activation pass, int8 codes between the layers, prepared
weights, CUDA-graph replay: all bit-identical logits; BN folded into the
convolutions: its own tolerance) are reported under `forms`.

Prints ONE JSON line (rank 0). The other benchmark configurations (single
layers, the quantizer sweep, the column-sharded fixed-point affine) follow
under `other_configs`; the keys a reader needs first are the last ones.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

IMAGE = (3, 224, 224)
CLASSES = 1000


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--batch", type=int, default=256, help="images per step over all GPUs")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (profiling runs)")
    ap.add_argument("--no-extras", action="store_true", help="skip the other configurations")
    ap.add_argument("--no-forms", action="store_true", help="skip the other execution forms of the network")
    ap.add_argument("--only-extras", action="store_true",
                    help="run only the other configurations and print their JSON (profiling runs)")
    ap.add_argument("--small-extras", action="store_true",
                    help="reduced sizes for the other configurations (ncu captures must stay small)")
    ap.add_argument("--sweep-max-log2", type=int, default=30, help="largest size of the quantizer sweep")
    ap.add_argument("--case", default=None, choices=sorted(KERNEL_CASES),
                    help="run one small single-kernel case a few times and exit (what the ncu captures under "
                         "profiles/ run; prints its CUDA-event time)")
    return ap.parse_args()


# --------------------------------------------------------------------------- single-kernel cases
def _case_folded_conv(C, HW, batch=256, residual=True):
    def make():
        import torch
        from nnabla_b200 import functions as F
        torch.manual_seed(0)
        w = torch.randn(C, C, 3, 3, device="cuda") * 0.1
        prep = F.prepare_binary_weights(w, 1, 1.0)
        scale, bias = (prep.alpha * 0.0625).contiguous(), torch.randn(C, device="cuda") * 0.1
        slots = F.codes_nhwc_slots(C)
        x = torch.randint(0, 128, (batch, HW * HW, slots), device="cuda", dtype=torch.int8)
        r = torch.randint(0, 128, (batch, HW * HW, slots), device="cuda", dtype=torch.int8)
        kw = dict(residual_codes=r, residual_delta=0.0625) if residual else {}
        return lambda: F.convolution_codes_folded(x, (batch, C, HW, HW), prep, scale, bias, (1, 1), (1, 1), (1, 1), **kw)
    return make


def _case_stem(codes, batch=256):
    def make():
        import torch
        from nnabla_b200 import functions as F
        torch.manual_seed(0)
        x = torch.randn(batch, 3, 224, 224, device="cuda")
        w, b = torch.randn(64, 3, 7, 7, device="cuda") * 0.1, torch.randn(64, device="cuda") * 0.1
        if codes:
            return lambda: F.convolution_relu_fixed_point_codes(x, w, b, (3, 3), (2, 2))
        return lambda: F.convolution(x, w, None, 1, (3, 3), (2, 2), (1, 1), 1)
    return make


def _case_quantizers(log2n):
    def make():
        import torch
        from nnabla_b200 import functions as F
        x = torch.rand(1 << log2n, device="cuda") * 8 - 4
        y = torch.empty_like(x)
        one = lambda v: torch.tensor([v], device="cuda")
        q = (one(-4.0), one(4.0), one(0.0), one(255.0))

        def run():
            F.fixed_point_quantize(x, True, 8, 2.0 ** -4, outputs=[y])
            F.pow2_quantize(x, True, True, 8, 1, outputs=[y])
            F.min_max_quantize(x, *q, outputs=[y])
        return run
    return make


def _case_quantizer_backward(log2n):
    def make():
        import torch
        from nnabla_b200 import functions as F
        n = 1 << log2n
        x, dy = torch.rand(n, device="cuda") * 9 - 4.5, torch.randn(n, device="cuda")
        dx = torch.empty_like(x)
        one = lambda v: torch.tensor([v], device="cuda")
        q = (one(-4.0), one(4.0), one(0.0), one(255.0))
        F.min_max_quantize(x, *q)

        def run():
            F.fixed_point_quantize_backward(x, dy, True, 8, 2.0 ** -4, True, False, dx)
            F.pow2_quantize_backward(x, dy, True, True, 8, 1, True, False, dx)
            F.min_max_quantize_backward(x, *q, dy, grads=(dx, None, None))
        return run
    return make


def _case_int8_gemm(n):
    def make():
        import torch
        from nnabla_b200 import functions as F
        x, w, b = torch.randn(n, n, device="cuda"), 0.02 * torch.randn(n, n, device="cuda"), torch.zeros(n, device="cuda")
        _, xc = F.fixed_point_quantize_with_codes(x, True, 8, 2.0 ** -5)
        _, wc = F.fixed_point_quantize_with_codes(w, True, 8, 2.0 ** -10)
        wk = F.transpose_codes(wc)
        return lambda: F.affine_from_kmajor_codes(xc, wk, n, 2.0 ** -5, 2.0 ** -10, b)
    return make


def _case_bwconv_f32act(batch):
    def make():
        import torch
        from nnabla_b200 import functions as F
        x = torch.relu(torch.randn(batch, 256, 28, 28, device="cuda"))
        w = torch.randn(256, 256, 3, 3, device="cuda") * (2.0 / 2304) ** 0.5
        wb, al = torch.zeros_like(w), torch.zeros(256, device="cuda")
        return lambda: F.binary_weight_convolution(x, w, wb, al, None, 1, (1, 1), (1, 1))
    return make


def _case_bwconv_fixed_point_act(batch, C=64, HW=56):
    """BinaryWeightConvolution as the graph calls it after a FixedPointQuantize: fp32 multiples of 2^-4 in,
    fp32 out; two kernels (operands in one launch, then the int8 contraction)."""
    def make():
        import torch
        from nnabla_b200 import functions as F
        torch.manual_seed(0)
        x = torch.randint(0, 128, (batch, C, HW, HW), device="cuda").float() * 0.0625
        w = torch.randn(C, C, 3, 3, device="cuda") * (2.0 / (9 * C)) ** 0.5
        wb, al = torch.zeros_like(w), torch.zeros(C, device="cuda")
        y = torch.empty(batch, C, HW, HW, device="cuda")
        return lambda: F.binary_weight_convolution(x, w, wb, al, None, 1, (1, 1), (1, 1), outputs=[y],
                                                   fixed_point_delta=0.0625)
    return make


def _case_fused_codes_pass(batch):
    def make():
        import torch
        from nnabla_b200 import functions as F
        a = torch.randn(batch, 64, 56, 56, device="cuda")
        bn = [torch.randn(64, device="cuda") * 0.1, 1 + 0.1 * torch.randn(64, device="cuda"),
              torch.randn(64, device="cuda") * 0.1, 0.5 + torch.rand(64, device="cuda")]
        return lambda: F.bn_add_relu_fixed_point_codes(a, bn)
    return make


KERNEL_CASES = {
    "folded_conv_64_56x56": _case_folded_conv(64, 56),
    "folded_conv_128_28x28": _case_folded_conv(128, 28),
    "folded_conv_256_14x14": _case_folded_conv(256, 14),
    "stem_codes": _case_stem(True),
    "stem_float": _case_stem(False),
    "quantizers_2p26": _case_quantizers(26),
    "quantizer_backward_2p26": _case_quantizer_backward(26),
    "int8_gemm_4096": _case_int8_gemm(4096),
    "bwconv_f32_activations_batch16": _case_bwconv_f32act(16),
    "bwconv_fixed_point_activations_64_56x56_batch192": _case_bwconv_fixed_point_act(192),
    "fused_codes_pass_batch128": _case_fused_codes_pass(128),
}


def run_case(name):
    import torch
    from nnabla_b200 import _capi as C
    torch.cuda.set_device(0)
    C.call("nb200_check_device")
    fn = KERNEL_CASES[name]()
    print(json.dumps({"case": name, "ms": float("%.5g" % time_gpu(fn, 5, warm=3))}))


def round_floats(o, digits=5):
    """Numbers with a few significant digits keep the JSON line short."""
    if isinstance(o, float):
        return float("%.*g" % (digits, o))
    if isinstance(o, dict):
        return {k: round_floats(v, digits) for k, v in o.items()}
    if isinstance(o, (list, tuple)):
        return [round_floats(v, digits) for v in o]
    return o


# --------------------------------------------------------------------------- CPU arm
def cpu_network():
    """(kind, function namespace) of the CPU implementation of the network's functions: the
    reference's own compiled code where oracle/_ref is present, else the C restatement."""
    from oracle import ops, ref
    if ref.available():
        return "reference", ops.reference()
    return "port", ops


def cpu_images_per_second(images, threads):
    """Runs the reference network on `images` images, one image per call, spread over `threads`
    host threads (independent function instances; the reference's CPU functions are
    single-threaded). Returns (images per second, seconds)."""
    from nnabla_b200 import resnet18
    kind, ns = cpu_network()
    params = resnet18.init_parameters(np.random.RandomState(0))
    rng = np.random.RandomState(1)
    xs = [rng.randn(1, *IMAGE).astype(np.float32) for _ in range(images)]
    cz = lambda w, shape=None: np.zeros(shape or w.shape, np.float32)

    def work(mine):
        net = resnet18.Runner(ns, params, cz, None, fixed_point_hint=False)
        for x in mine:
            net(x)
    t0 = time.perf_counter()
    ths = [threading.Thread(target=work, args=(xs[i::threads],)) for i in range(threads)]
    for t in ths:
        t.start()
    for t in ths:
        t.join()
    dt = time.perf_counter() - t0
    return kind, images / dt, dt


def run_reference_arm(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    threads = min(os.cpu_count() or 1, 16)
    for _ in range(1 if args.warmup > 0 else 0):
        cpu_images_per_second(threads, threads)
    total, kind = 0.0, "port"
    for _ in range(args.steps):
        kind, _, dt = cpu_images_per_second(threads, threads)
        total += dt
    value = threads * args.steps / total
    sample = "each step: %d images (of the %d of a batch), one per host thread, whole network per image" % (
        threads, args.batch)
    line = {
        "impl": "reference", "metric": "resnet18_images_per_sec", "value": value, "unit": "images/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.batch, args.gpus),
        "cpu_baseline": {"value": value, "unit": "images/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(round_floats(line)))


def workload_config(batch, world):
    return {"workload": "configs[4]: binary-weight ResNet-18 forward, fp32 input [%d,3,224,224], 1000 classes, "
                        "random init, batch sharded over the GPUs" % batch,
            "global_batch": batch, "images_per_gpu": batch // max(1, world),
            "form": "graph as written, one call per function"}


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


def measure_int8_peak(seconds=2.0):
    """Dense int8 tensor-core throughput of this GPU with the library GEMM (torch._int_mm, 8192^3),
    by the method of the measured bf16 peak: best of 10 single launches, and back to back for a
    few seconds (sustained, under the power cap). TOP/s."""
    import torch
    n = 8192
    a = torch.randint(-127, 128, (n, n), device="cuda", dtype=torch.int8)
    b = torch.randint(-127, 128, (n, n), device="cuda", dtype=torch.int8).t()  # column-major, as the library wants
    ops = 2.0 * n ** 3
    for _ in range(3):
        torch._int_mm(a, b)
    best = 1e30
    for _ in range(10):
        best = min(best, time_gpu(lambda: torch._int_mm(a, b), 1, warm=0))
    per = max(best, 1e-3)
    iters = max(10, int(seconds * 1e3 / per))
    sustained = time_gpu(lambda: torch._int_mm(a, b), iters, warm=0)
    return {"int8_tops": ops / best / 1e9, "int8_tops_sustained": ops / sustained / 1e9,
            "how": "torch._int_mm 8192^3, best of 10 and %d launches back to back" % iters}


class FunctionTimer:
    """Wraps a function namespace: every call is bracketed by CUDA events on the current stream
    and filed under the function's name with its algorithmic work (bytes for the memory-bound
    functions, operations for the contractions)."""

    def __init__(self, ns):
        self._ns = ns
        self.records = []

    def __getattr__(self, name):
        import torch
        fn = getattr(self._ns, name)

        def timed(*a, **kw):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            y = fn(*a, **kw)
            e1.record()
            self.records.append((name, e0, e1, self._work(name, a, kw, y)))
            return y
        return timed

    @staticmethod
    def _work(name, a, kw, y):
        from nnabla_b200 import functions as lib
        n_in = a[0].numel()
        n_out = y.numel() if hasattr(y, "numel") else 0
        if name == "fixed_point_quantize":
            # a quantizer that also left int8 codes with its result wrote one byte more per value
            with_codes = lib._sideband_get(y, a[3] if len(a) > 3 else kw.get("delta", 2 ** -4)) is not None
            return ("bytes", (9.0 if with_codes else 8.0) * n_in)
        if name in ("batch_normalization", "relu"):
            return ("bytes", 8.0 * n_in)
        if name == "add2":
            return ("bytes", 12.0 * n_in)
        if name in ("max_pooling", "global_average_pooling"):
            return ("bytes", 4.0 * (n_in + n_out))
        if name in ("convolution", "binary_weight_convolution"):
            w = a[1]
            k = w.shape[1] * w.shape[2] * w.shape[3]
            kind = "int8_ops" if (name == "binary_weight_convolution" and kw.get("fixed_point_delta")) else "flops"
            # the function as the graph calls it also moves its fp32 input and result (and reads the weights,
            # and writes their signs): with quantized activations that traffic, not the contraction, is the
            # larger floor for most layers
            extra = 2 if name == "binary_weight_convolution" else 1
            # an input that carries its quantizer's codes is read as one byte per value
            from_codes = (name == "binary_weight_convolution" and kw.get("fixed_point_delta") is not None
                          and lib._sideband_get(a[0], kw["fixed_point_delta"]) is not None)
            return (kind, 2.0 * n_out * k, (1.0 if from_codes else 4.0) * n_in + 4.0 * (n_out + extra * w.numel()))
        if name == "affine":
            return ("flops", 2.0 * n_out * a[1].shape[0])
        return ("bytes", 0.0)

    def table(self):
        import torch
        torch.cuda.synchronize()
        fam = {}
        for name, e0, e1, rec in self.records:
            kind, work = rec[0], rec[1]
            f = fam.setdefault(name, {"calls": 0, "ms": 0.0, "kind": kind, "work": 0.0, "bytes": 0.0})
            f["calls"] += 1
            f["ms"] += e0.elapsed_time(e1)
            f["work"] += work
            f["bytes"] += rec[2] if len(rec) > 2 else (work if kind == "bytes" else 0.0)
        return fam


# DRAM bytes of the 19 binary-weight convolutions of one pass at 256 images, from one ncu capture of this file's
# own command line (dram__bytes_read.sum + dram__bytes_write.sum over their 38 kernels: 812 MB read, 794 MB
# written; lines of a result that were still in L2 when its kernel ended are not in the write figure; 15 of the
# 19 read their quantizer's int8 codes, not the fp32 tensor). The tensors of the pass grow in proportion to the
# images, so other batch sizes scale it (below 2^23 values per tensor the quantizers leave no codes and the
# convolutions read fp32: the figure is then low).
NCU_DRAM_BYTES_BINARY_WEIGHT_CONVOLUTIONS_AT_256 = 1605.9e6


def function_table(F, params, gz, x, peaks, int8_peak, passes=3):
    """Per-function time table of the as-written graph (each function's calls bracketed by CUDA
    events, averaged over `passes` forward passes) and the roofline entry of the family with the
    largest share."""
    from nnabla_b200 import resnet18
    timer = FunctionTimer(F)
    net = resnet18.Runner(timer, params, gz, codes_sideband=True)
    net(x)
    timer.records.clear()
    for _ in range(passes):
        net(x)
    fam = timer.table()
    total = sum(f["ms"] for f in fam.values())
    rows = {}
    for name, f in sorted(fam.items(), key=lambda kv: -kv[1]["ms"]):
        ms = f["ms"] / passes
        row = {"calls": f["calls"] // passes, "ms": ms, "share": f["ms"] / total}
        if f["kind"] == "bytes":
            row["GBps"] = f["work"] / f["ms"] / 1e6
            row["frac_hbm"] = row["GBps"] / peaks["hbm_gbs"]
        elif f["kind"] == "int8_ops":
            row["int8_tops"] = f["work"] / f["ms"] / 1e9
            row["frac_int8"] = row["int8_tops"] / int8_peak
        else:
            row["tflops"] = f["work"] / f["ms"] / 1e9
            row["frac_bf16"] = row["tflops"] / peaks["bf16_tflops"]
        if f["kind"] != "bytes" and f["bytes"] > 0:
            row["GBps_fp32_tensors"] = f["bytes"] / f["ms"] / 1e6
            row["frac_hbm"] = row["GBps_fp32_tensors"] / peaks["hbm_gbs"]
        rows[name] = row
    top = max(fam.items(), key=lambda kv: kv[1]["ms"])
    name, f = top
    per_call_ms = f["ms"] / f["calls"]
    tensor_peak = int8_peak if f["kind"] == "int8_ops" else peaks["bf16_tflops"]
    # the bound of a function is the larger of its two floors: moving its tensors, or its operations
    t_hbm = f["bytes"] / peaks["hbm_gbs"] / 1e6
    t_tensor = 0.0 if f["kind"] == "bytes" else f["work"] / tensor_peak / 1e9
    if t_hbm >= t_tensor:
        ach, peak, unit, bound, work = f["bytes"] / f["ms"] / 1e6, peaks["hbm_gbs"], "GB/s", "hbm", f["bytes"]
    else:
        unit = "TOP/s" if f["kind"] == "int8_ops" else "TFLOP/s"
        ach, peak, bound, work = f["work"] / f["ms"] / 1e9, tensor_peak, "tensor", f["work"]
    traffic = None
    if name == "binary_weight_convolution":
        traffic = NCU_DRAM_BYTES_BINARY_WEIGHT_CONVOLUTIONS_AT_256 * int(x.shape[0]) / 256.0 / (f["calls"] / passes)
    roof = {"bound": bound, "kernel": name, "achieved": ach, "peak": peak, "unit": unit, "frac": ach / peak,
            "traffic": traffic, "traffic_note": "bytes per call, ncu capture of one pass at 256 images scaled by images",
            "share_of_step": f["ms"] / total, "ms_per_call": per_call_ms,
            "algorithmic_work_per_call": work / f["calls"],
            "floors_ms_per_pass": {"hbm": t_hbm / passes, "tensor": t_tensor / passes}}
    # the whole step against the sum of every function's larger floor
    step_floor = 0.0
    for g in fam.values():
        tp = int8_peak if g["kind"] == "int8_ops" else peaks["bf16_tflops"]
        step_floor += max(g["bytes"] / peaks["hbm_gbs"] / 1e6, 0.0 if g["kind"] == "bytes" else g["work"] / tp / 1e9)
    roof["step_floor_ms"] = step_floor / passes
    roof["step_ms_sum_of_functions"] = total / passes
    roof["step_frac_of_floor"] = step_floor / total
    return rows, roof


def run_extras(args, rank, world, peaks, int8_peak):
    """The other configurations, timed per rank (inputs resident in HBM)."""
    import torch
    import torch.distributed as dist
    from nnabla_b200 import functions as F
    from nnabla_b200 import sharding
    out = {}
    gen = torch.Generator(device="cuda").manual_seed(99 + rank)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=gen)

    def maxr(ms):
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return ms

    # configs[0]: BinaryWeightAffine 256 x 1024 x 4096 (replicated on every rank; working set fits L2)
    M, K, N = 256, 1024, 4096
    x, w, b = rn(M, K), 0.02 * rn(K, N), torch.zeros(N, device="cuda")
    wb, al = torch.zeros_like(w), torch.zeros(N, device="cuda")
    ms = maxr(time_gpu(lambda: F.binary_weight_affine(x, w, wb, al, b), 50))
    e0 = {"ms": ms, "us_hbm_floor": 38.8e6 / peaks["hbm_gbs"] / 1e3, "frac_hbm": 38.8e6 / peaks["hbm_gbs"] / 1e6 / ms,
          "tflops_issued_bf16x3": 6 * M * K * N / ms / 1e9, "frac_bf16_issued": 6 * M * K * N / ms / 1e9 / peaks["bf16_tflops"]}
    try:  # the same forward_impl recorded once as a CUDA graph
        from nnabla_b200 import graphs
        cap0 = graphs.Captured(lambda xx: F.binary_weight_affine(xx, w, wb, al, b), x)
        e0["ms_cuda_graph"] = maxr(time_gpu(lambda: cap0.graph.replay(), 50))
        del cap0
    except RuntimeError as e:
        e0["ms_cuda_graph"] = None
    out["configs[0] binary_weight_affine 256x1024x4096"] = e0

    # configs[1]: quantizer sweep, 2^20 .. 2^30 elements (sizes up to L2 run out of L2 after the first pass)
    one = lambda v: torch.tensor([v], device="cuda", dtype=torch.float32)
    qa, qb, la, lb = one(-4.0), one(4.0), one(0.0), one(255.0)
    sweep = {}
    for k in range(20, min(args.sweep_max_log2, 22 if args.small_extras else 30) + 1, 2):
        n = 1 << k
        xs = torch.rand(n, device="cuda", generator=gen) * 8 - 4
        ys = torch.empty_like(xs)
        it = 50 if k <= 24 else (20 if k <= 28 else 10)
        t = [maxr(time_gpu(lambda: F.fixed_point_quantize(xs, True, 8, 2.0 ** -4, outputs=[ys]), it)),
             maxr(time_gpu(lambda: F.pow2_quantize(xs, True, True, 8, 1, outputs=[ys]), it)),
             maxr(time_gpu(lambda: F.min_max_quantize(xs, qa, qb, la, lb, outputs=[ys]), it))]
        sweep["2^%d" % k] = {"GBps_fxp_pow2_minmax": [8.0 * n / v / 1e6 for v in t],
                             "frac_hbm": [8.0 * n / v / 1e6 / peaks["hbm_gbs"] for v in t]}
        del xs, ys
    out["configs[1] quantizers (per GPU)"] = sweep
    torch.cuda.empty_cache()

    # configs[2]: 8-bit fixed-point affine, output columns sharded over the ranks
    M, K, N = (4096, 4096, 4096) if args.small_extras else (8192, 4096, 8192)
    Ns = N // world
    x = rn(M, K)
    w = 0.02 * rn(K, Ns)
    b = 0.01 * rn(Ns)
    xq, xc = F.fixed_point_quantize_with_codes(x, True, 8, 2.0 ** -5)
    wq, wc = F.fixed_point_quantize_with_codes(w, True, 8, 2.0 ** -10)
    ops = 2.0 * M * K * N
    ms_gemm = maxr(time_gpu(lambda: F.affine_from_codes(xc, wc, 2.0 ** -5, 2.0 ** -10, b), 20))
    wk = F.transpose_codes(wc)  # the weight's codes in the tensor core's layout, made once per weight update
    ms_prepared = maxr(time_gpu(lambda: F.affine_from_kmajor_codes(xc, wk, K, 2.0 ** -5, 2.0 ** -10, b), 20))

    def chain():  # what a graph runs: FixedPointQuantize(x), FixedPointQuantize(W), Affine on the fp32 tensors
        a = F.fixed_point_quantize(x, True, 8, 2.0 ** -5)
        c = F.fixed_point_quantize(w, True, 8, 2.0 ** -10)
        return F.affine(a, c, b, fixed_point=(2.0 ** -5, 2.0 ** -10))
    ms_chain = maxr(time_gpu(chain, 10))
    ms_qx = maxr(time_gpu(lambda: F.fixed_point_quantize(x, True, 8, 2.0 ** -5), 10))
    ms_qw = maxr(time_gpu(lambda: F.fixed_point_quantize(w, True, 8, 2.0 ** -10), 10))
    ms_aff = maxr(time_gpu(lambda: F.affine(xq, wq, b, fixed_point=(2.0 ** -5, 2.0 ** -10)), 10))
    e2 = {"columns_per_gpu": Ns,
          "ms_gemm_kmajor_codes": ms_prepared, "int8_tops_kmajor_codes": ops / ms_prepared / 1e9,
          "frac_int8_kmajor_codes": ops / world / ms_prepared / 1e9 / int8_peak,
          "ms_gemm_codes": ms_gemm, "int8_tops_codes": ops / ms_gemm / 1e9,
          "frac_int8_codes": ops / world / ms_gemm / 1e9 / int8_peak,
          "ms_chain_quantize_x_quantize_w_affine": ms_chain, "int8_tops_chain": ops / ms_chain / 1e9,
          "frac_int8_chain": ops / world / ms_chain / 1e9 / int8_peak,
          "ms_quantize_x": ms_qx, "ms_quantize_w": ms_qw, "ms_affine_on_fp32_operands": ms_aff}
    try:  # the library's int8 GEMM on the same codes, for context (int32 output, no scaling, no bias)
        wct = wc.t().contiguous().t()
        ms_lib = maxr(time_gpu(lambda: torch._int_mm(xc, wct), 20))
        e2["ms_library_int8_gemm"] = ms_lib
    except Exception:  # noqa: BLE001 - the comparison is optional
        e2["ms_library_int8_gemm"] = None
    if world > 1:
        def gemm_and_gather():
            yy = F.affine_from_codes(xc, wc, 2.0 ** -5, 2.0 ** -10, b)
            return sharding.gather_columns(yy, N)
        e2["ms_gemm_plus_nccl_allgather"] = maxr(time_gpu(gemm_and_gather, 10))
        # the gather fused into the contraction: every rank's epilogue stores its slab into all ranks'
        # [M, N] results over NVLink (peer mappings), then one tiny all-reduce orders the ranks
        mats = sharding.PeerMatrices(M, N)

        def gemm_fused_gather():
            F.affine_from_codes_gather(xc, wc, 2.0 ** -5, 2.0 ** -10, b, mats.ptrs, rank, N, rank * Ns)
            mats.fence()
        e2["ms_gemm_fused_gather_all_ranks"] = maxr(time_gpu(gemm_fused_gather, 10))
        e2["fused_gather_GBps_out_per_gpu"] = (world - 1) * M * Ns * 4 / e2["ms_gemm_fused_gather_all_ranks"] / 1e6
        # gather to rank 0 only: every rank stores its slab into rank 0's result (and rank 0 into its own)
        only0 = [mats.ptrs[0]]

        def gemm_gather_rank0():
            F.affine_from_codes_gather(xc, wc, 2.0 ** -5, 2.0 ** -10, b, only0, 0, N, rank * Ns)
            mats.fence()
        try:
            e2["ms_gemm_fused_gather_rank0"] = maxr(time_gpu(gemm_gather_rank0, 10))
        except Exception as exc:  # noqa: BLE001
            e2["ms_gemm_fused_gather_rank0"] = None
            e2["gather_rank0_note"] = str(exc)[:60]
        gemm_fused_gather()
        torch.cuda.synchronize()
        want = gemm_and_gather()
        same = bool(torch.equal(mats.local, want))
        # a window of rows of the gathered result against an integer product worked out on its own:
        # every partial sum is an integer below 2^24, so fp32(acc) * 2^-15 + bias is exact up to one rounding
        rows = slice(M // 2 - 16, M // 2 + 16)
        acc = xc[rows].to(torch.float64) @ wc.to(torch.float64)  # exact: |acc| < 2^53
        ref = (acc.to(torch.float32) * (2.0 ** -15) + b)
        window_ok = bool(torch.equal(mats.local[rows, rank * Ns:(rank + 1) * Ns], ref))
        flags = torch.tensor([int(same), int(window_ok)], device="cuda")
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)
        e2["fused_gather_equals_allgather"] = bool(flags[0].item())
        e2["gathered_rows_equal_integer_product"] = bool(flags[1].item())
        mats.close()
        assert e2["fused_gather_equals_allgather"], "peer-store gather differs from the NCCL all-gather"
        assert e2["gathered_rows_equal_integer_product"], "gathered result differs from the integer product"
    out["configs[2] fixed-point int8 affine %dx%dx%d" % (M, K, N)] = e2
    del x, w, xq, wq, xc, wc, wk
    torch.cuda.empty_cache()

    # configs[3]: BinaryWeightConvolution 3x3, 256 -> 256, 28 x 28, batch 128 sharded over the ranks
    Nb = max(1, (16 if args.small_extras else 128) // world)
    x = torch.relu(rn(Nb, 256, 28, 28))
    w = rn(256, 256, 3, 3) * (2.0 / 2304) ** 0.5
    wb, al, b = torch.zeros_like(w), torch.zeros(256, device="cuda"), torch.zeros(256, device="cuda")
    ms = maxr(time_gpu(lambda: F.binary_weight_convolution(x, w, wb, al, b, 1, (1, 1), (1, 1)), 10))
    flops = 2.0 * (Nb * world * 28 * 28) * 256 * 2304
    e3 = {"ms": ms, "images_per_gpu": Nb, "tflops_algorithmic": flops / ms / 1e9,
          "tflops_issued_fp16x2": 2 * flops / ms / 1e9,
          "frac_f16_issued_per_gpu": 2 * flops / world / ms / 1e9 / peaks["bf16_tflops"]}
    dyc = rn(Nb, 256, 28, 28)
    gxc, gwc, gbc = torch.empty_like(x), torch.empty_like(w), torch.empty(256, device="cuda")
    e3["ms_backward_dx"] = maxr(time_gpu(lambda: F.binary_weight_convolution_backward(
        x, wb, al, dyc, 1, (1, 1), (1, 1), propagate_down=(True, False, False), grads=(gxc, None, None)), 10))
    e3["ms_backward_dw_db"] = maxr(time_gpu(lambda: F.binary_weight_convolution_backward(
        x, wb, al, dyc, 1, (1, 1), (1, 1), propagate_down=(False, True, True), grads=(None, gwc, gbc)), 10))
    out["configs[3] binary_weight_convolution 3x3 256->256 28x28 batch %d" % (Nb * world)] = e3
    del x, w, dyc, gxc
    torch.cuda.empty_cache()
    return out


def run_b200_arm(args):
    import torch
    import torch.distributed as dist
    from nnabla_b200 import _capi as C
    from nnabla_b200 import functions as F
    from nnabla_b200 import graphs, resnet18

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

    def maxr(v):
        if world > 1:
            t = torch.tensor([v], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return v

    peaks, peak_kind = measured_peaks()
    int8 = measure_int8_peak(0.5 if args.small_extras else 2.0)
    int8_peak = int8["int8_tops"]

    if args.only_extras:
        extras = run_extras(args, rank, world, peaks, int8_peak)
        if rank == 0:
            print(json.dumps(round_floats({"measured_int8_peak": int8, "other_configs": extras})))
        if world > 1:
            dist.destroy_process_group()
        return

    assert args.batch % world == 0, "the batch must divide over the GPUs"
    Bg = args.batch // world
    params = {k: torch.from_numpy(v).cuda() for k, v in resnet18.init_parameters(np.random.RandomState(0)).items()}
    # this rank's images of the seeded batch, in pinned host memory
    hx = torch.from_numpy(np.random.RandomState(1000 + rank).randn(Bg, *IMAGE).astype(np.float32)).pin_memory()
    x = hx.cuda()
    gz = lambda t, shape=None: torch.zeros(shape or tuple(t.shape), device="cuda")
    # every FixedPointQuantize of a large tensor also leaves its int8 channel-last codes with its result, and the
    # binary-weight convolutions called on that result read them (same functions, same results bit for bit)
    net = resnet18.Runner(F, params, gz, codes_sideband=True)

    # ---- the timed region: K forward passes of the graph as written ------------------------
    # The calls of one forward pass (one C-ABI call per reference function) are recorded once into a CUDA
    # graph and replayed: the same kernels in the same order, without the host's per-call cost, which at a
    # few dozen images per GPU would otherwise bound the step. If the capture fails the calls run eagerly.
    W = max(args.warmup, 3)
    for _ in range(W):
        net(x)
    F.check_device_status()
    captured, calls_per_pass = None, None
    try:
        c0 = C.calls_made()
        captured = graphs.Captured(net, x, warmup=1)
        calls_per_pass = (C.calls_made() - c0) // 2  # one warm-up pass and the captured one
        step = captured.graph.replay
    except RuntimeError:
        captured = None
        step = lambda: net(x)
    for _ in range(W):
        step()
    F.check_device_status()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    barrier()
    calls0 = C.calls_made()
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record()
    for _ in range(args.steps):
        step()
    t_end.record()
    barrier()
    clocks = sampler.stop() if sampler else None
    calls = C.calls_made() - calls0 if captured is None else calls_per_pass * args.steps
    elapsed_ms = maxr(t_start.elapsed_time(t_end))
    F.check_device_status()
    value = args.batch * args.steps / (elapsed_ms / 1e3)
    logits = (captured.static_output if captured is not None else net(x)).clone()
    finite = bool(torch.isfinite(logits).all())

    # ---- end to end: pinned host images in, logits out, every step -------------------------
    e2e = None
    if not args.no_e2e:
        copy_stream = torch.cuda.Stream()
        hy = [torch.empty(Bg, CLASSES, dtype=torch.float32).pin_memory() for _ in range(2)]
        main = torch.cuda.current_stream()
        # two input buffers in turn; with the forward captured, each buffer is the static input of its own graph
        caps = None
        if captured is not None:
            try:
                caps = [captured, graphs.Captured(net, x, warmup=1)]
            except RuntimeError:
                caps = None
        xin = [c.static_inputs[0] for c in caps] if caps else [torch.empty_like(x), torch.empty_like(x)]

        def e2e_run(steps):
            done = [None, None]
            for s in range(steps):
                k = s & 1
                with torch.cuda.stream(copy_stream):
                    if done[k] is not None:
                        copy_stream.wait_event(done[k])  # the buffer's previous step has finished with it
                    xin[k].copy_(hx, non_blocking=True)
                    ready = torch.cuda.Event()
                    ready.record(copy_stream)
                main.wait_event(ready)
                if caps:
                    caps[k].graph.replay()
                    y = caps[k].static_output
                else:
                    y = net(xin[k])
                hy[k].copy_(y, non_blocking=True)
                done[k] = torch.cuda.Event()
                done[k].record(main)
            torch.cuda.synchronize()
        e2e_run(2)
        barrier()
        t0 = time.perf_counter()
        e2e_run(args.steps)
        barrier()
        e2e_s = maxr(time.perf_counter() - t0)
        e2e = {"value": args.batch * args.steps / e2e_s, "unit": "images/s",
               "h2d_bytes_per_step": world * Bg * int(np.prod(IMAGE)) * 4, "d2h_bytes_per_step": world * Bg * CLASSES * 4,
               "steps": args.steps, "ms_per_step": 1e3 * e2e_s / args.steps,
               "api": "resnet18.Runner over nnabla_b200.functions%s; pinned host images -> device (copy of step s+1 "
                      "overlaps the forward of step s) -> logits to pinned host memory"
                      % (", its calls replayed from a CUDA graph" if caps else "")}
        del xin, caps

    # ---- the other execution forms of the same graph ---------------------------------------
    forms = None
    if not args.no_forms:
        forms = {"as_written_ms": elapsed_ms / args.steps,
                 "as_written_is_cuda_graph_replay": captured is not None}
        same = True

        def form(key, runner, iters=5):
            nonlocal same
            ms = maxr(time_gpu(lambda: runner(x), iters, warm=2))
            F.check_device_status()
            forms[key + "_ms"] = ms
            forms[key + "_images_per_sec"] = args.batch / ms * 1e3
            return runner
        same_as = lambda r: bool(torch.equal(r(x), logits))
        same &= same_as(form("as_written_call_by_call", net))
        same &= same_as(form("as_written_without_quantizer_codes_call_by_call", resnet18.Runner(F, params, gz)))
        same &= same_as(form("fused_activation_pass", resnet18.Runner(F, params, gz, fused=True)))
        same &= same_as(form("int8_codes_between_layers", resnet18.Runner(F, params, gz, fused="codes")))
        prep = form("int8_codes_prepared_weights", resnet18.Runner(F, params, gz, fused="codes", prepared_weights=True))
        same &= same_as(prep)
        try:
            cap_codes = graphs.Captured(prep, x)
            same &= same_as(form("cuda_graph_replay", cap_codes))
            del cap_codes
        except RuntimeError as e:  # a capture another thread's CUDA call interrupted: report, do not fail the run
            forms["cuda_graph_replay_ms"] = None
        if hasattr(resnet18, "FoldedRunner"):
            folded = resnet18.FoldedRunner(F, params)
            form("bn_folded_int8_epilogue", folded)
            fl = folded(x)
            try:
                cap_folded = graphs.Captured(folded, x)
                form("bn_folded_cuda_graph_replay", cap_folded)
                del cap_folded
            except RuntimeError:
                forms["bn_folded_cuda_graph_replay_ms"] = None
            forms["bn_folded_logits_rel_rms_vs_as_written"] = float(
                ((fl - logits).double().pow(2).mean() / logits.double().pow(2).mean()).sqrt())
            forms["bn_folded_top1_agreement"] = float((fl.argmax(1) == logits.argmax(1)).float().mean())
        # the same graph through nnabla's own graph engine with the extension backend: built with
        # CgVariable / CgFunction / connect(), run by CgVariable::forward(clear_buffer=true) on "b200:float"
        from nnabla_b200 import nbla_graph
        if nbla_graph.available():
            hostp = {k: v.cpu().numpy() for k, v in params.items()}
            g = nbla_graph.Graph("b200:float", str(local))
            xv = g.variable(hx.numpy())
            cz = lambda w, shape=None: np.zeros(shape or w.shape, np.float32)
            yv = resnet18.Runner(g, hostp, cz, None, fixed_point_hint=False)(xv)
            g.forward(yv, clear_buffer=True, repeat=2)
            nbla_graph.reset_counters()
            sec = maxr(g.forward(yv, clear_buffer=True, repeat=5))
            forms["nnabla_graph_engine_b200_context_ms"] = 1e3 * sec
            forms["nnabla_graph_engine_b200_context_images_per_sec"] = args.batch / sec
            forms["nnabla_graph_engine_int8_convolutions_per_pass"] = nbla_graph.counter("int8_convolutions") / 5
            same &= bool(np.array_equal(g.data(yv), logits.cpu().numpy()))
            g.close()
            nbla_graph.clear_memory_cache()
            # one training step of the same network through the same engine: forward with batch statistics,
            # backward with clear_buffer (every function's backward pass on the b200 backend)
            try:
                gt = nbla_graph.Graph("b200:float", str(local), need_grad=True)
                yt = resnet18.Runner(gt, {k: v.copy() for k, v in hostp.items()}, cz, None, fixed_point_hint=False,
                                     batch_stat=True)(gt.variable(hx.numpy()))
                dyt = np.random.RandomState(7).randn(Bg, CLASSES).astype(np.float32)
                leaves = gt.parameter_leaves()

                def train_step():
                    t0 = time.perf_counter()
                    gt.forward(yt, clear_buffer=False)
                    for _, v in leaves:
                        gt.zero_grad(v)
                    gt.backward(yt, dyt, clear_buffer=True)
                    return time.perf_counter() - t0
                train_step()
                sec = maxr(min(train_step() for _ in range(3)))
                forms["nnabla_graph_engine_training_step_ms"] = 1e3 * sec
                forms["nnabla_graph_engine_training_images_per_sec"] = args.batch / sec
                gt.close()
            except RuntimeError as e:
                forms["nnabla_graph_engine_training_step_ms"] = None
                forms["nnabla_graph_engine_training_error"] = str(e)[:200]
            nbla_graph.clear_memory_cache()
            torch.cuda.set_device(local)
        flag = torch.tensor([int(same)], device="cuda")
        if world > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        forms["bit_identical_logits_all_forms"] = bool(flag.item())

    # ---- per-function table and the roofline entry -----------------------------------------
    table, roofline = function_table(F, params, gz, x, peaks, int8_peak)
    roofline["peak_source"] = peak_kind if roofline["unit"] != "TOP/s" else "measured in this run (torch._int_mm 8192^3)"
    if roofline["bound"] == "hbm" and roofline["kernel"].endswith("convolution"):
        roofline["bytes_counted"] = ("input of every call (int8 codes where its quantizer left them, else fp32), fp32 "
                                     "result, weights read, their signs written")

    del x, logits
    torch.cuda.empty_cache()
    extras = None
    if not args.no_extras:
        extras = run_extras(args, rank, world, peaks, int8_peak)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    cpu_baseline = None
    if not args.no_cpu_baseline:
        n_img = 24  # about 12 s of one host thread
        kind, ips, dt = cpu_images_per_second(n_img, 1)
        cpu_baseline = {"value": ips, "unit": "images/s", "cores": 1, "kind": kind,
                        "sample": "%d images of the batch, whole network per image, 1 thread (%.1f s)" % (n_img, dt)}
    line = {
        "other_configs": extras,
        "measured_int8_peak": int8,
        "functions": table,
        "forms": forms,
        "metric": "resnet18_images_per_sec", "value": value, "unit": "images/s", "n_gpus": world, "steps": args.steps,
        "warmup": W, "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": dict(workload_config(args.batch, world),
                       execution=("the pass's C-ABI calls recorded once into a CUDA graph and replayed" if captured
                                  is not None else "call by call"),
                       quantizer_codes="FixedPointQuantize of tensors of 2^23 values and more leaves int8 channel-last codes "
                                       "with its result; the binary-weight convolution called on it reads them",
                       l2="per-step activations (over 800 MB at 256 images) exceed L2; no flush needed"),
        "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "clocks": clocks,
        "gpu_launches": calls, "gpu_launches_note": "C-ABI calls whose kernels ran in the timed region (replayed from the CUDA graph when "
                                                "config.execution says so); each launches 1 to 4 kernels",
        "logits_finite": finite,
    }
    print(json.dumps(round_floats(line)))
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.case:
        run_case(args.case)
        return
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_b200_arm(args)


if __name__ == "__main__":
    main()
