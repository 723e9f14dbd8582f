#!/usr/bin/env python
"""Benchmark of the DCNv4 operator hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: a "sweep" is one DCNv4 forward and one backward at each of the four FlashInternImage-T
stage shapes (N=64 per GPU; (H=W, C, G) = (56,64,4), (28,128,8), (14,256,16), (7,512,32);
group_channels 16, 3x3 / stride 1 / pad 1), in fp32 and in fp16: 16 operator calls.  All eight
forwards run first, then all eight backwards, so the ~1 GB of distinct tensors a sweep touches
passes through between two uses of any buffer (inputs larger than the 126 MB L2; no explicit
flush).  A "step" is SWEEPS_PER_STEP sweeps back to back (one sweep is ~2 ms, too short a timed
region for clock sampling at 20 steps).  Data is synthetic (seeded, the distributions the
configuration states).

`value` = algorithmic bytes of a step (each tensor counted once) x ranks / device time, inputs
resident in HBM, calls made straight through the C ABI.  `e2e` = the same step through the public
autograd API with pinned HOST buffers: host->device copies of every input and device->host
copies of every result inside the timed region.  `roofline` describes the operator call that
takes the most device time.  `cpu_baseline` times the reference's own pure-PyTorch (grid_sample-based)
core on the host cores -- a bounded sample of the same workload plus benchmark configuration 0 --
falling back to a restatement of the same algorithm when the reference file is not available.

Multi-GPU (torchrun, one rank per GPU): the batch is sharded, every rank runs the same step on
its own N=64 shard, there is no data-path collective; timing is barrier + synchronize on both
sides, max over ranks (weak scaling).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

STAGES = ((56, 64, 4), (28, 128, 8), (14, 256, 16), (7, 512, 32))
N_PER_GPU = 64
D = 16
METRIC = "dcnv4_fwd_bwd_hbm_throughput"
UNIT = "GB/s"
WORKLOAD = "dcnv4_fwd+bwd sweep, FlashInternImage-T stage shapes, N=64/GPU, fp32+fp16"
CPU_SAMPLE_N = 8
# One sweep of the 16 operator calls takes ~2 ms: too short a timed region for the clock sampler when the
# driver asks for 20 steps.  A step is therefore SWEEPS_PER_STEP sweeps back to back; bytes scale with it.
SWEEPS_PER_STEP = 8
# dram__bytes_read.sum + dram__bytes_write.sum per operator call, from one ncu capture of each stage-1
# kernel at N=64 (kernel only; for the fp16 backward plus the zero-fill of the fp32 accumulation buffer,
# 51.4 MB, and the convert pass, 51.4 + 25.7 MB, which ncu was not asked to capture)
NCU_TRAFFIC_BYTES = {
    "dcnv4_fwd_56x56x64_fp32": 171.1e6, "dcnv4_fwd_56x56x64_fp16": 77.2e6,
    "dcnv4_bwd_56x56x64_fp32": 348.7e6, "dcnv4_bwd_56x56x64_fp16": 200.9e6 + 128.5e6,
}
MODEL_GLOBAL_BATCH = 256
MODEL_ITERS = 10


def algorithmic_bytes(N, HW, C, G, es):
    K = 9
    Ppad = -(-3 * G * K // 8) * 8
    fwd = es * (N * HW * HW * C + N * HW * HW * Ppad + N * HW * HW * C)
    bwd = es * (2 * N * HW * HW * C + 2 * N * HW * HW * Ppad + N * HW * HW * C)
    return fwd, bwd


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


# ----------------------------------------------------------------------------- clocks

class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self, t0, t1):
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        rows = [r for ts, r in self.rows if t0 - 0.05 <= ts <= t1 + 0.15] or [r for _, r in self.rows]
        for r in rows:
            parts = [p.strip() for p in r.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


# ----------------------------------------------------------------------------- CPU arm

def _cpu_model():
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.lower().startswith("model name"):
                    return line.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown"


def _cpu_callable():
    """(fwd(t, G), fwd_bwd(t, G), kind): the reference's own pure-PyTorch core, imported unmodified
    (oracle/ref_core.py), when its file is mounted or installed under oracle/_ref; otherwise the
    grid_sample restatement of the same algorithm (oracle/torch_core.py)."""
    a = (3, 3, 1, 1, 1, 1, 1, 1)
    try:
        from oracle import ref_core
        if ref_core.available():
            core = ref_core.load()
            return (lambda t, G: ref_core.dcnv4_forward(core, t["value"], t["offset_mask"], *a, G, D, 1.0, 0),
                    lambda t, G: ref_core.dcnv4_forward_backward(core, t["value"], t["offset_mask"], t["grad_out"],
                                                                 *a, G, D, 1.0, 0),
                    "reference")
    except Exception as exc:  # a broken install must not take the benchmark down
        _note(f"reference core unavailable ({type(exc).__name__}: {exc}); timing the restatement")
    from oracle import torch_core
    return (lambda t, G: torch_core.dcnv4_core(t["value"], t["offset_mask"], *a, G, D, 1.0, 0),
            lambda t, G: torch_core.dcnv4_fwd_bwd(t["value"], t["offset_mask"], t["grad_out"], *a, G, D, 1.0, 0),
            "port")


def _median_time(fn, reps, warm):
    for _ in range(warm):
        fn()
    ts = []
    for _ in range(reps):
        t0 = time.perf_counter()
        fn()
        ts.append(time.perf_counter() - t0)
    return statistics.median(ts)


def cpu_baseline(reps=5, warm=2):
    """The reference's pure-PyTorch (grid_sample-based) core on the host cores, fp32, all threads:
      * the bounded sample of the benchmark step: the four stage shapes at N=CPU_SAMPLE_N, forward +
        autograd backward -> GB/s of algorithmic bytes (the line's metric);
      * benchmark configuration 0 (N=2, 56x56x64, G=4, seed 0): forward alone and forward + backward.
    Returns the `cpu_baseline` object of the JSON line."""
    import torch
    from oracle import inputs as oin
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    fwd, fwd_bwd, kind = _cpu_callable()
    tensors, nbytes = [], 0
    for HW, C, G in STAGES:
        tensors.append((oin.dcnv4_inputs(CPU_SAMPLE_N, HW, HW, G, D, seed=HW), G))
        f, b = algorithmic_bytes(CPU_SAMPLE_N, HW, C, G, 4)
        nbytes += f + b

    def sweep():
        for t, G in tensors:
            fwd_bwd(t, G)

    med = _median_time(sweep, reps, warm)
    t0 = oin.dcnv4_inputs(2, 56, 56, 4, D, seed=0)
    f0, b0 = algorithmic_bytes(2, 56, 64, 4, 4)
    with torch.no_grad():
        fwd_s = _median_time(lambda: fwd(t0, 4), max(reps, 10), warm)
    fb_s = _median_time(lambda: fwd_bwd(t0, 4), max(reps, 10), warm)
    name = ("dcnv3_core_pytorch of the reference (classification/ops_dcnv3/functions/dcnv3_func.py), unmodified"
            if kind == "reference" else "grid_sample restatement of the reference's pure-PyTorch core")
    desc = (f"{name}; 4 stage shapes at N={CPU_SAMPLE_N} (1/{N_PER_GPU // CPU_SAMPLE_N} of the batch), fp32 only, "
            f"forward + autograd backward, median of {reps} passes")
    return {"value": nbytes / med / 1e9, "unit": UNIT, "cores": torch.get_num_threads(), "kind": kind,
            "sample": desc, "ms_per_pass": med * 1e3, "cpu_model": _cpu_model(),
            "config0": {"shape": "N=2, 56x56x64, G=4x16, 3x3/s1/p1, fp32, seed 0",
                        "fwd_ms": fwd_s * 1e3, "fwd_gbs": f0 / fwd_s / 1e9,
                        "fwd_bwd_ms": fb_s * 1e3, "fwd_bwd_gbs": (f0 + b0) / fb_s / 1e9}}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    cb = cpu_baseline(reps=max(1, args.steps), warm=max(1, min(args.warmup, 3)))
    line = {
        "impl": "reference", "metric": METRIC, "value": cb["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": cb["ms_per_pass"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": cb["sample"]},
        "cpu_baseline": cb,
        "e2e": {"value": cb["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


# ----------------------------------------------------------------------------- GPU arm

def synthetic_inputs(torch, N, HW, G, seed, dtype, dev):
    """value ~N(0,1); per group 18 offsets ~N(0,1) px then 9 masks ~U(0,1), pad columns zero;
    grad_out ~N(0,1).  Seeded on the CPU generator, then cast and moved."""
    g = torch.Generator().manual_seed(seed)
    K, C = 9, G * D
    Ppad = -(-3 * G * K // 8) * 8
    value = torch.randn(N, HW, HW, C, generator=g)
    off = torch.randn(N, HW, HW, G, 2 * K, generator=g)
    msk = torch.rand(N, HW, HW, G, K, generator=g)
    om = torch.zeros(N, HW, HW, Ppad)
    om[..., : 3 * G * K] = torch.cat((off, msk), -1).reshape(N, HW, HW, 3 * G * K)
    gout = torch.randn(N, HW, HW, C, generator=g)
    return tuple(x.to(device=dev, dtype=dtype) for x in (value, om, gout))


class Case:
    """Device-resident tensors of one (stage, dtype) and its raw C-ABI calls."""

    def __init__(self, torch, lib, HW, C, G, dtype, code, seed, dev):
        self.HW, self.C, self.G, self.code, self.dtype = HW, C, G, code, dtype
        self.value, self.om, self.gout = synthetic_inputs(torch, N_PER_GPU, HW, G, seed, dtype, dev)
        self.out = torch.empty_like(self.value)
        self.gvalue = torch.empty_like(self.value)
        self.gom = torch.empty_like(self.om)
        self.ws_bytes = lib.dcnv4b200_bwd_workspace_bytes(code, N_PER_GPU, HW, HW, G, D)
        self.ws = torch.empty(max(self.ws_bytes, 16) // 4, dtype=torch.float32, device=dev)
        es = self.value.element_size()
        self.fwd_bytes, self.bwd_bytes = algorithmic_bytes(N_PER_GPU, HW, C, G, es)
        self.lib = lib
        self.name = f"{HW}x{HW}x{C}_{'fp32' if code == 0 else 'fp16'}"
        self.scalars = (N_PER_GPU, HW, HW, G, D, 3, 3, 1, 1, 1, 1, 1, 1, 1.0, 0, self.om.shape[-1], 0)
        self.kernels_fwd = 1
        self.kernels_bwd = 1 + (1 if self.ws_bytes else 0)

    def fwd(self, stream):
        rc = self.lib.dcnv4b200_fwd(self.value.data_ptr(), self.om.data_ptr(), self.out.data_ptr(),
                                    self.code, *self.scalars, stream)
        assert rc == 0, rc

    def bwd(self, stream):
        rc = self.lib.dcnv4b200_bwd(self.value.data_ptr(), self.om.data_ptr(), self.gout.data_ptr(),
                                    self.gvalue.data_ptr(), self.gom.data_ptr(),
                                    self.ws.data_ptr() if self.ws_bytes else None, self.ws_bytes,
                                    self.code, *self.scalars, stream)
        assert rc == 0, rc


def time_reference_cuda(torch, cases, reps=5):
    """Per operator call: median device time of the reference CUDA extension (its own launch
    specs), L2 flushed between runs, plus max |difference| to our result on the same inputs.
    Returns None when the extension has not been built."""
    try:
        from oracle import ref_cuda
        if not ref_cuda.available():
            return None
        ref_cuda.ext()
    except Exception as exc:  # missing build, ABI mismatch, ...
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}
    flush = torch.empty(256 * 1024 * 1024 // 4, device=cases[0].value.device)
    out = []
    for c in cases:
        a = (3, 3, 1, 1, 1, 1, 1, 1, c.G, D, 1.0, 0)
        stream = torch.cuda.current_stream().cuda_stream
        c.fwd(stream)
        c.bwd(stream)
        for which in ("fwd", "bwd"):
            fn = ((lambda: ref_cuda.dcnv4_forward(c.value, c.om, *a)) if which == "fwd" else
                  (lambda: ref_cuda.dcnv4_backward(c.value, c.om, c.gout, *a)))
            try:
                res = fn()
                torch.cuda.synchronize()
            except Exception as exc:
                out.append({"op": f"dcnv4_{which}_{c.name}", "error": f"{type(exc).__name__}: {exc}"[:160]})
                continue
            ts = []
            for _ in range(reps):
                flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1))
            if which == "fwd":
                diff = (res.float() - c.out.float()).abs().max().item()
            else:
                diff = max((res[0].float() - c.gvalue.float()).abs().max().item(),
                           (res[1].float() - c.gom.float()).abs().max().item())
            nbytes = c.fwd_bytes if which == "fwd" else c.bwd_bytes
            ms = statistics.median(ts)
            out.append({"op": f"dcnv4_{which}_{c.name}", "ms": ms, "gbs": nbytes / ms / 1e6,
                        "max_abs_diff_vs_ours": diff})
            del res
    return out


def time_flash_deform_attn(torch, lib, dev, with_reference, reps=5):
    """FlashDeformAttn forward/backward at the Deformable-DETR encoder shape (8 images, 8 heads x 32
    channels, 4 levels x 4 points per level), in both readings of the configuration's level sizes:
    100x152, 50x76, 25x38, 13x19 (20,197 positions, the reference script's) and 100x150, 50x75, 25x38,
    13x19 (19,947 positions); fp32 and fp16: median device time per call through the C ABI, L2 flushed
    between runs, and the reference CUDA extension on the same tensors when it is available."""
    out = []
    for levels in (((100, 152), (50, 76), (25, 38), (13, 19)), ((100, 150), (50, 75), (25, 38), (13, 19))):
        out += _time_flash_deform_attn_levels(torch, lib, dev, levels, with_reference, reps)
    return out


def _time_flash_deform_attn_levels(torch, lib, dev, levels, with_reference, reps):
    B, G, Dh, K, L = 8, 8, 32, 4, 4
    shapes = torch.tensor(levels, dtype=torch.int64, device=dev)
    sizes = shapes[:, 0] * shapes[:, 1]
    starts = torch.cat((sizes.new_zeros(1), sizes.cumsum(0)[:-1]))
    Len = int(sizes.sum())
    g = torch.Generator().manual_seed(7)
    value32 = torch.randn(B, Len, G, Dh, generator=g)
    sla32 = torch.cat((torch.rand(B, Len, G, 2 * L * K, generator=g), torch.randn(B, Len, G, L * K, generator=g)), -1)
    gout32 = torch.randn(B, Len, G * Dh, generator=g)
    flush = torch.empty(256 * 1024 * 1024 // 4, device=dev)
    ref = None
    if with_reference:
        try:
            from oracle import ref_cuda
            ref = ref_cuda if ref_cuda.available() and ref_cuda.ext() is not None else None
        except Exception:
            ref = None
    stream = torch.cuda.current_stream().cuda_stream
    out = []

    def timed(fn):
        fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(reps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts)

    for dtype, code, tag in ((torch.float32, 0, "fp32"), (torch.float16, 1, "fp16")):
        v, sla, go = (x.to(device=dev, dtype=dtype) for x in (value32, sla32, gout32))
        es = v.element_size()
        y, gv, gs = torch.empty(B, Len, G * Dh, dtype=dtype, device=dev), torch.empty_like(v), torch.empty_like(sla)
        ws_bytes = lib.fdab200_bwd_workspace_bytes(code, B, Len, G, Dh)
        ws = torch.empty(max(ws_bytes, 16) // 4, dtype=torch.float32, device=dev)
        fwd_bytes = es * (v.numel() + sla.numel() + y.numel())
        bwd_bytes = fwd_bytes + es * (v.numel() + sla.numel())

        def fwd():
            rc = lib.fdab200_fwd(v.data_ptr(), shapes.data_ptr(), starts.data_ptr(), sla.data_ptr(), y.data_ptr(),
                                 code, B, Len, G, Dh, L, Len, K, stream)
            assert rc == 0, rc

        def bwd():
            rc = lib.fdab200_bwd(v.data_ptr(), shapes.data_ptr(), starts.data_ptr(), sla.data_ptr(), go.data_ptr(),
                                 gv.data_ptr(), gs.data_ptr(), ws.data_ptr() if ws_bytes else None, ws_bytes,
                                 code, B, Len, G, Dh, L, Len, K, stream)
            assert rc == 0, rc

        for which, fn, nbytes in (("fwd", fwd, fwd_bytes), ("bwd", bwd, bwd_bytes)):
            ms = timed(fn)
            row = {"op": f"fda_{which}_8x{Len}x8x32_{tag}", "ms": ms, "bytes": nbytes, "gbs": nbytes / ms / 1e6}
            if ref is not None:
                try:
                    rfn = ((lambda: ref.fda_forward(v, shapes, starts, sla, K)) if which == "fwd" else
                           (lambda: ref.fda_backward(v, shapes, starts, sla, go, K)))
                    row["reference_cuda_ms"] = timed(rfn)
                    res = rfn()
                    if which == "fwd":
                        row["max_abs_diff_vs_reference"] = (res.float() - y.float()).abs().max().item()
                    else:
                        row["max_abs_diff_vs_reference"] = max((res[0].float() - gv.float()).abs().max().item(),
                                                               (res[1].float() - gs.float()).abs().max().item())
                    del res
                except Exception as exc:
                    row["reference_cuda_error"] = f"{type(exc).__name__}: {exc}"[:160]
            out.append(row)
        del v, sla, go, y, gv, gs, ws
    return out


def time_config0(torch, lib, dev, reps=200):
    """Benchmark configuration 0 (N=2, 56x56x64, G=4, fp32, seed 0) on the GPU through the C ABI: device
    time per forward and per forward + backward, launches back to back (the tensors fit L2 many times
    over; this is the latency of a small call, reported beside the CPU core's time for the same call)."""
    value, om, gout = synthetic_inputs(torch, 2, 56, 4, 0, torch.float32, dev)
    out, gv, gom = torch.empty_like(value), torch.empty_like(value), torch.empty_like(om)
    sc = (2, 56, 56, 4, D, 3, 3, 1, 1, 1, 1, 1, 1, 1.0, 0, om.shape[-1], 0)
    stream = torch.cuda.current_stream().cuda_stream

    def fwd():
        assert lib.dcnv4b200_fwd(value.data_ptr(), om.data_ptr(), out.data_ptr(), 0, *sc, stream) == 0

    def bwd():
        assert lib.dcnv4b200_bwd(value.data_ptr(), om.data_ptr(), gout.data_ptr(), gv.data_ptr(), gom.data_ptr(),
                                 None, 0, 0, *sc, stream) == 0

    def timed(fn):
        for _ in range(10):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    f_ms = timed(fwd)
    fb_ms = timed(lambda: (fwd(), bwd()))
    fb, bb = algorithmic_bytes(2, 56, 64, 4, 4)
    return {"shape": "N=2, 56x56x64, G=4x16, 3x3/s1/p1, fp32, seed 0", "fwd_ms": f_ms, "fwd_gbs": fb / f_ms / 1e6,
            "fwd_bwd_ms": fb_ms, "fwd_bwd_gbs": (fb + bb) / fb_ms / 1e6, "launches_back_to_back": reps}


def time_fused_offset(torch, dev, batch=256, reps=20):
    """The DCNv4 module's inference path around the operator at the four FlashInternImage-T stage shapes,
    fp16: value projection + forward that computes its offset/mask rows itself, against both projections
    as one product + stand-alone forward.  Each two-kernel sequence is captured in a CUDA graph (as the
    model's forward is) and replayed `reps` times between two events; at batch 256 the tensors of one
    replay exceed L2 at the first two stages."""
    from dcnv4_b200 import ops
    rows = []
    for side, C, G in STAGES:
        P, h = (27 * G + 7) // 8 * 8, torch.float16
        gen = torch.Generator(device=dev).manual_seed(side)
        x = torch.randn(batch, side * side, C, device=dev, generator=gen).to(h)
        wv = (torch.randn(C, C, device=dev, generator=gen) / C ** 0.5).to(h)
        wo = (torch.randn(P, C, device=dev, generator=gen) / C ** 0.5).to(h)
        bv, bo = torch.zeros(C, device=dev, dtype=h), torch.randn(P, device=dev, generator=gen).to(h)
        wcat, bcat = torch.cat([wv, wo]).contiguous(), torch.cat([bv, bo]).contiguous()

        def two_step():
            v, om = ops.linear_pair_forward(x, wcat, bcat, C)
            return ops.dcnv4_forward(v.view(batch, side, side, C), om.view(batch, side, side, P), 3, 3, 1, 1, 1, 1,
                                     1, 1, G, D, 1.0, 256, 0)

        def fused():
            v = ops.linear_forward(x, wv, bv)
            return ops.dcnv4_fused_offset_forward(v.view(batch, side, side, C), x, wo, bo, G, D, 1.0)

        def timed(fn):
            side_stream = torch.cuda.Stream(device=dev)
            side_stream.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side_stream):
                for _ in range(3):
                    fn()
            torch.cuda.current_stream(dev).wait_stream(side_stream)
            torch.cuda.synchronize(dev)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                fn()
            for _ in range(3):
                graph.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                graph.replay()
            e1.record()
            torch.cuda.synchronize(dev)
            return e0.elapsed_time(e1) / reps

        same = bool(torch.equal(two_step(), fused()))
        rows.append({"shape": f"{batch}x{side}x{side}x{C}, G={G}", "two_step_ms": timed(two_step),
                     "fused_ms": timed(fused), "bit_identical": same})
    return rows


def _note(msg):
    """Progress note on stderr (stdout carries only the JSON line)."""
    if os.environ.get("RANK", "0") == "0":
        print(f"[bench] {msg}", file=sys.stderr, flush=True)


def time_model_with_reference_kernels(torch, model, images, iters=5):
    """ms per forward of `model` with the reference CUDA extension as the DCNv4 core, stock LayerNorm,
    nn.Linear / nn.GELU / separate additions and no CUDA graph; None when the extension is not built."""
    try:
        from oracle import ref_cuda
        if not ref_cuda.available():
            return None
        ref_cuda.ext()
    except Exception:
        return None
    from dcnv4_b200 import flash_intern_image as fii
    from dcnv4_b200 import ops as our_ops
    from dcnv4_b200.modules import dcnv4 as dcn_mod

    class RefCore:
        @staticmethod
        def apply(x, om, kh, kw, sh, sw, ph, pw, dh, dw, G, Dg, scale, step, rc):
            return ref_cuda.dcnv4_forward(x, om, kh, kw, sh, sw, ph, pw, dh, dw, G, Dg, scale, rc, step)

    saved_fn, saved_flag, saved_fused = dcn_mod.DCNv4Function, fii.LayerNorm.use_library_kernel, our_ops.FUSED_LINEAR
    dcn_mod.DCNv4Function, fii.LayerNorm.use_library_kernel, our_ops.FUSED_LINEAR = RefCore, False, False
    try:
        with torch.no_grad():
            for _ in range(2):
                model(images)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                model(images)
            e1.record()
            torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters
    except Exception as exc:
        _note(f"reference-stack model leg failed: {type(exc).__name__}: {exc}")
        return None
    finally:
        dcn_mod.DCNv4Function, fii.LayerNorm.use_library_kernel, our_ops.FUSED_LINEAR = saved_fn, saved_flag, saved_fused


def run_ours(args):
    import torch
    import torch.distributed as dist

    from dcnv4_b200 import DCNv4Function, _lib

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # NCCL writes its version / debug lines to stdout by default; stdout is reserved for the JSON line
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.lib()

    cases = []
    for si, (HW, C, G) in enumerate(STAGES):
        for dtype, code in ((torch.float32, 0), (torch.float16, 1)):
            cases.append(Case(torch, lib, HW, C, G, dtype, code, seed=1000 * rank + si, dev=dev))
    stream = torch.cuda.current_stream().cuda_stream
    ops = [(c, "fwd") for c in cases] + [(c, "bwd") for c in cases]
    if args.case:  # profiling aid: only the operator calls whose name contains the given text
        ops = [(c, w) for c, w in ops if args.case in f"dcnv4_{w}_{c.name}"]
        if not ops:
            raise SystemExit(f"--case {args.case!r} matches no operator call")

    step_bytes = sum(c.fwd_bytes if w == "fwd" else c.bwd_bytes for c, w in ops)
    launches_per_step = sum(c.kernels_fwd if w == "fwd" else c.kernels_bwd for c, w in ops)

    sweeps = 1 if args.case else SWEEPS_PER_STEP

    def step(events=None):
        # the per-call events bracket the first sweep of a step; the others run unobserved
        for rep in range(sweeps):
            for i, (c, which) in enumerate(ops):
                if events is not None and rep == 0:
                    events[i][0].record()
                (c.fwd if which == "fwd" else c.bwd)(stream)
                if events is not None and rep == 0:
                    events[i][1].record()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    _note(f"world {world}: {len(ops)} operator calls per step, warming up")
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()

    ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in ops]
          for _ in range(args.steps)]
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    wall0 = time.time()
    t_start.record()
    for k in range(args.steps):
        step(ev[k])
    t_end.record()
    barrier()
    wall1 = time.time()
    elapsed_ms = t_start.elapsed_time(t_end)
    _note(f"timed region done: {elapsed_ms / args.steps:.3f} ms per step")

    # ---- end to end through the public autograd API with pinned host buffers
    host_in, host_out = [], []
    for c in ([] if (args.no_e2e or args.case) else cases):
        host_in.append([x.cpu().pin_memory() for x in (c.value, c.om, c.gout)])
        host_out.append([torch.empty_like(x, device="cpu").pin_memory() for x in (c.out, c.gvalue, c.gom)])
    h2d = sum(x.numel() * x.element_size() for xs in host_in for x in xs)
    d2h = sum(x.numel() * x.element_size() for xs in host_out for x in xs)

    # Three streams: uploads, compute, downloads.  PCIe is full duplex, so while one operator call
    # computes, the next call's inputs are already arriving and the previous call's results are
    # already leaving; events carry the dependencies, and record_stream keeps the caching allocator
    # from recycling a buffer another stream still reads.
    up, down = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    # Order of the 8 (stage, dtype) cases inside an end-to-end sweep.  Uploads run back to back on one
    # stream and downloads on another, one case behind; a sweep therefore lasts (all uploads) + max(first
    # upload, last download).  The two smallest cases go to the ends, the large ones in between.
    by_size = sorted(range(len(host_in)), key=lambda i: sum(x.numel() * x.element_size() for x in host_in[i]))
    e2e_order = ([by_size[0]] + by_size[2:] + [by_size[1]]) if len(by_size) > 2 else by_size

    def e2e_step():
        main = torch.cuda.current_stream(dev)
        up.wait_stream(main)
        for c, hin, hout in ((cases[i], host_in[i], host_out[i]) for i in e2e_order):
            with torch.cuda.stream(up):
                v = hin[0].to(dev, non_blocking=True)
                om = hin[1].to(dev, non_blocking=True)
                go = hin[2].to(dev, non_blocking=True)
                arrived = torch.cuda.Event()
                arrived.record(up)
            main.wait_event(arrived)
            for t in (v, om, go):
                t.record_stream(main)
            v.requires_grad_(True)
            om.requires_grad_(True)
            out = DCNv4Function.apply(v, om, 3, 3, 1, 1, 1, 1, 1, 1, c.G, D, 1.0, 256, 0)
            out.backward(go)
            computed = torch.cuda.Event()
            computed.record(main)
            down.wait_event(computed)
            with torch.cuda.stream(down):
                for dst, src in zip(hout, (out.detach(), v.grad, om.grad)):
                    src.record_stream(down)
                    dst.copy_(src, non_blocking=True)
        main.wait_stream(down)

    e2e_steps = max(1, min(args.steps, 10))
    e2e_ms = float("nan")
    if not args.no_e2e and not args.case:
        for _ in range(2):
            e2e_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(e2e_steps):
            e2e_step()
        e1.record()
        barrier()
        e2e_ms = e0.elapsed_time(e1)
    # ---- the caller of the hot path: FlashInternImage-T inference, random-init weights, fp16,
    #      batch sharded over the ranks (global batch 256), no collective
    model_ms, model_batch = float("nan"), max(1, MODEL_GLOBAL_BATCH // world)
    model_weak_ms = float("nan")    # N > 1 only: the same forward with the full batch on every GPU
    model_ref_ms = None
    if not args.no_model and not args.case:
        import copy
        from dcnv4_b200.flash_intern_image import GraphedInference, flash_intern_image, fold_batchnorm_
        torch.manual_seed(0)
        model = flash_intern_image("t").to(dev).half().eval()
        folded = fold_batchnorm_(copy.deepcopy(model))

        def time_graphed(batch):
            # inference form: BatchNorms folded into their convolutions, one CUDA graph per forward
            imgs = torch.randn(batch, 3, 224, 224, device=dev, dtype=torch.float16)
            graphed = GraphedInference(folded, imgs)
            for _ in range(3):
                graphed(imgs)
            barrier()
            m0, m1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            m0.record()
            for _ in range(MODEL_ITERS):
                graphed(imgs)
            m1.record()
            barrier()
            return m0.elapsed_time(m1) / MODEL_ITERS, imgs

        model_ms, images = time_graphed(model_batch)
        if world > 1:
            model_weak_ms, _ = time_graphed(MODEL_GLOBAL_BATCH)
        del folded
        # the same network the way the reference stack executes it: eager launches, torch.nn.LayerNorm,
        # and the reference's own CUDA operator (oracle/_ref) in place of ours.  Baseline leg, rank 0 only.
        if rank == 0 and world == 1 and not args.no_ref_cuda:
            model_ref_ms = time_model_with_reference_kernels(torch, model, images)
        del model, images
    # ---- the reference's own CUDA kernels, recompiled unmodified for sm_100 (oracle/build_ref.py),
    #      timed beside ours on the same tensors: "the kernel to beat".  Baseline leg only.
    ref_cuda_ops = None
    if rank == 0 and world == 1 and not args.case and not args.no_ref_cuda:
        ref_cuda_ops = time_reference_cuda(torch, cases)
    fda_ops = None
    if rank == 0 and world == 1 and not args.case and not args.no_fda:
        fda_ops = time_flash_deform_attn(torch, lib, dev, with_reference=not args.no_ref_cuda)
    config0 = time_config0(torch, lib, dev) if rank == 0 and not args.case else None
    fused_rows = time_fused_offset(torch, dev) if rank == 0 and world == 1 and not args.case and not args.no_model else None
    if rank == 0:
        sampler.stop()

    _note("all legs done, reducing times over ranks")
    times = torch.tensor([elapsed_ms, e2e_ms, model_ms, model_weak_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms, model_ms, model_weak_ms = times.tolist()

    if rank == 0:
        per_op = []
        for i, (c, which) in enumerate(ops):
            ms = statistics.mean(ev[k][i][0].elapsed_time(ev[k][i][1]) for k in range(args.steps))
            nbytes = c.fwd_bytes if which == "fwd" else c.bwd_bytes
            per_op.append({"op": f"dcnv4_{which}_{c.name}", "ms": ms, "bytes": nbytes,
                           "gbs": nbytes / ms / 1e6,
                           "launches": c.kernels_fwd if which == "fwd" else c.kernels_bwd})
        peak, peak_kind = peaks()
        # The roofline entry is about one kernel: only calls that are a single kernel launch qualify
        # (a 16-bit backward call is the kernel plus the convert pass, so its event time is not a
        # launch duration; its kernel is the same template and a few microseconds shorter).
        dom = max((o for o in per_op if o["launches"] == 1), key=lambda o: o["ms"])
        for o in per_op:
            o["frac"] = o["gbs"] / peak
        value = step_bytes * sweeps * world * args.steps / elapsed_ms / 1e6
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32+f16 storage, f32 arithmetic",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "batch_per_gpu": N_PER_GPU, "global_batch": N_PER_GPU * world,
                       "parallelism": f"batch-sharded x{world}, no collective",
                       "l2": "inputs larger than L2: a step touches ~1 GB of distinct tensors between two "
                             "uses of any buffer (all forwards, then all backwards); no explicit flush",
                       "sweeps_per_step": sweeps, "operator_calls_per_step": len(ops) * sweeps,
                       "bytes_per_step_per_gpu": step_bytes * sweeps},
            "e2e": {"value": step_bytes * world * e2e_steps / e2e_ms / 1e6, "unit": UNIT,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "ms_per_step": e2e_ms / e2e_steps, "sweeps_per_step": 1,
                    "api": "dcnv4_b200.DCNv4Function.apply + backward, pinned host buffers, "
                           "uploads / compute / downloads on three streams, smallest cases first and last"},
            "gpu_launches": launches_per_step * sweeps * args.steps,
            "roofline": {"bound": "hbm", "kernel": dom["op"], "achieved": dom["gbs"], "peak": peak,
                         "peak_kind": peak_kind, "unit": "GB/s", "frac": dom["gbs"] / peak, "traffic": NCU_TRAFFIC_BYTES.get(dom["op"]),
                         "ms": dom["ms"], "algorithmic_bytes": dom["bytes"]},
            "ops": per_op,
            "clocks": sampler.summary(wall0, wall1),
            "config0_gpu": config0,
            "reference_cuda": ref_cuda_ops,
            "flash_deform_attn": fda_ops,
            "fused_offset_forward": fused_rows,
            "flash_intern_image_t": None if model_ms != model_ms else {
                "img_per_s": model_batch * world / model_ms * 1e3, "ms_per_batch": model_ms,
                "batch_per_gpu": model_batch, "global_batch": model_batch * world, "dtype": "fp16",
                "input": "224x224 synthetic", "weights": "random init", "parallelism": f"batch-sharded x{world}",
                "img_per_s_with_full_batch_per_gpu": None if model_weak_ms != model_weak_ms else
                MODEL_GLOBAL_BATCH * world / model_weak_ms * 1e3,
                "execution": "BatchNorm folded into the convolutions, tensor-core Linear with fused GELU / "
                             "residual / LayerNorm, CUDA graph replay per forward, input copied into the graph's "
                             "buffer each iteration",
                "reference_stack_img_per_s": (model_batch / model_ref_ms * 1e3) if model_ref_ms else None,
                "reference_stack": "same network, eager launches, torch.nn.LayerNorm / Linear / GELU, reference "
                                   "CUDA operator (its forward is wrong at the 14x14 and 7x7 stages; timing only)"},
        }
        if args.case or args.no_e2e:
            line["e2e"] = None
        if world == 1 and not args.no_cpu_baseline and not args.case:
            line["cpu_baseline"] = cpu_baseline()
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


def run_train_l(args):
    """Optional workload (--workload train_l): FlashInternImage-L training step, random-init weights,
    1024x1024 synthetic images, batch 2 per GPU, bf16 autocast, activation checkpointing as in the
    released -L config, AdamW, DDP gradient all-reduce over NCCL when launched with torchrun, with the
    16-bit gradient compression hook the reference's trainer registers (classification/main.py:228-235;
    --grad-compress picks fp16 as there, bf16, fp32 or none).  Prints one JSON line with images/s
    (whole job, max step time over ranks) and, for N > 1, the step time with the gradient exchange
    switched off (DDP no_sync), whose difference is what the all-reduce costs after overlap."""
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    from dcnv4_b200.flash_intern_image import flash_intern_image

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(0)
    size, res, batch = args.train_size, args.train_res, 2
    model = flash_intern_image(size, with_cp=True).to(dev).train()
    hooked = False
    if world > 1:
        from dcnv4_b200 import ddp_hooks
        model = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local], broadcast_buffers=False,
                                                          gradient_as_bucket_view=True,
                                                          bucket_cap_mb=args.bucket_cap_mb)
        hooked = ddp_hooks.register(model, args.grad_compress)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4, weight_decay=0.05)
    g = torch.Generator(device="cpu").manual_seed(100 + rank)
    images = torch.randn(batch, 3, res, res, generator=g).to(dev)
    labels = torch.randint(0, 1000, (batch,), generator=g).to(dev)

    import contextlib

    def step(sync=True):
        opt.zero_grad(set_to_none=True)
        ctx = contextlib.nullcontext() if (sync or world == 1) else model.no_sync()
        with ctx:
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss = F.cross_entropy(model(images).float(), labels)
            loss.backward()
        opt.step()
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        loss = step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = step()
    e1.record()
    barrier()
    nosync_ms = float("nan")
    if world > 1:   # the same step without the gradient exchange (ranks drift apart: timing only)
        for _ in range(2):
            step(sync=False)
        barrier()
        n0, n1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n0.record()
        for _ in range(args.steps):
            step(sync=False)
        n1.record()
        barrier()
        nosync_ms = n0.elapsed_time(n1)
    t = torch.tensor([e0.elapsed_time(e1), nosync_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t[0].item() / args.steps
    nosync_ms = t[1].item() / args.steps
    n_params = sum(p.numel() for p in model.parameters())
    if rank == 0:
        print(json.dumps({
            "metric": f"flash_intern_image_{size}_train_throughput", "value": batch * world / ms * 1e3, "unit": "img/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 autocast",
            "data": "synthetic", "loss": float(loss.detach()),
            "config": {"workload": f"FlashInternImage-{size.upper()} training step, {res}x{res}, batch {batch}/GPU, "
                                   "AdamW, activation checkpointing, DDP all-reduce",
                       "global_batch": batch * world, "parallelism": f"dp{world}",
                       "grad_compress": args.grad_compress if hooked else "none",
                       "bucket_cap_mb": args.bucket_cap_mb if world > 1 else None},
            "ddp": None if world == 1 else {
                "ranks_in_process_group": dist.get_world_size(), "backend": dist.get_backend(),
                "gradient_bytes_fp32": n_params * 4,
                "wire_bytes_per_step": n_params * (2 if hooked and args.grad_compress in ("fp16", "bf16") else 4),
                "ms_per_step_without_gradient_exchange": nosync_ms,
                "allreduce_share_of_step": max(0.0, (ms - nosync_ms) / ms)},
            "peak_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30}), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end arm (profiling runs)")
    ap.add_argument("--no-model", action="store_true", help="skip the FlashInternImage-T throughput arm")
    ap.add_argument("--no-ref-cuda", action="store_true", help="skip timing the reference CUDA extension")
    ap.add_argument("--no-fda", action="store_true", help="skip the FlashDeformAttn (Deformable-DETR shape) leg")
    ap.add_argument("--case", default="", help="profiling aid: run only operator calls whose name contains "
                    "this text, e.g. fwd_56x56x64_fp32 (names are dcnv4_{fwd,bwd}_{HxWxC}_{fp32,fp16})")
    ap.add_argument("--workload", choices=("ops", "train_l"), default="ops",
                    help="ops (default): the DCNv4 operator sweep; train_l: FlashInternImage-L training step")
    ap.add_argument("--train-size", default="l", choices=("t", "s", "b", "l"))
    ap.add_argument("--grad-compress", default="fp16", choices=("none", "fp32", "fp16", "bf16"),
                    help="DDP gradient all-reduce wire format of --workload train_l (the reference registers fp16)")
    ap.add_argument("--bucket-cap-mb", type=int, default=100,
                    help="DDP gradient bucket size of --workload train_l (measured at 2 GPUs: 25 MB 147.8 ms per "
                         "step, 100 MB 138.3 ms, 400 MB 139.7 ms)")
    ap.add_argument("--train-res", type=int, default=1024)
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.workload == "train_l":
        return run_train_l(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
