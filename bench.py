#!/usr/bin/env python
"""Benchmark of the BoxConv2d forward+backward hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg5]

The default workload and the contract line are cfg5: the 1/8-frame ENet box block,
BoxConv2d(32, 4, 64, 128), on a GLOBAL batch of 256 samples that is divided over the GPUs (strong
scaling: 256 / 128 / 64 / 32 samples per GPU on 1 / 2 / 4 / 8 GPUs).  The line also carries a `cfg2`
key: the same block at 16 samples per GPU.  `--workload cfg2|cfg3|cfg1` time those shapes per GPU
(weak scaling), `--workload cfg4` the integral image alone, `--workload infer` the batch-1 inference
block tails of one frame.

One step = one training pass of the box block over one batch of synthetic input: parameter
clip, forward, backward (grad-input and the four parameter gradients) and, on more than one GPU,
the all-reduce of the packed (4, C, F) parameter gradient.  `value` is the whole job's output
elements per second: the median of at least 15 consecutive rounds of K steps (enough rounds for a
timed region of 0.3 s), each round between two CUDA events, per round the maximum over the ranks.
Every GPU count launches the same way: one CUDA graph replay per step.

The line printed by rank 0 carries, besides the contract keys:
  roofline      achieved HBM GB/s of the dominant kernel (algorithmic bytes / mean device time of
                that kernel, from per-kernel CUDA events recorded by the library during an eager
                repeat of K steps) against the measured copy bandwidth of this pool
  cpu_baseline  the reference's own CPU code on this machine's host cores (N=1 only)
  e2e           the same metric from pinned host buffers to host results through the module, and
                the floor that bare copies of the same bytes set
  clocks        SM clock and throttle reasons sampled through NVML during the timed rounds
  allreduce_check  (more than one GPU) the reduced gradients against the sum of the ranks' local
                gradients and every rank's shard against a full-batch run on rank 0; the run exits
                non-zero when they differ

`--impl reference` times the reference's CPU implementation of the same step (its compiled
extension built by oracle/build_ref.py; the plain-C oracle if that build is absent).
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "box-convolutions_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import numpy as np  # noqa: E402
import torch  # noqa: E402

from workloads import CONFIGS, make_workload  # noqa: E402

def stage(msg):
    """Progress line on stderr (rank 0 only) so that a stalled run shows where it stopped."""
    if os.environ.get("RANK", "0") == "0":
        print("[bench %.1fs] %s" % (time.perf_counter() - _T0, msg), file=sys.stderr, flush=True)


_T0 = time.perf_counter()


def arm_watchdog(seconds):
    """Ends the process from the host side if the run takes longer than `seconds` (a stuck
    collective or rendezvous must not keep a GPU box busy for its whole time limit)."""
    def fire():
        print("[bench] watchdog: no result after %d s, giving up" % seconds, file=sys.stderr, flush=True)
        os._exit(3)
    t = threading.Timer(seconds, fire)
    t.daemon = True
    t.start()
    return t


METRIC = "BoxConv2d fwd+bwd output Gelem/s"
UNIT = "Gelem/s"
BUFFER_SETS = 4          # rotated between steps so that the footprint exceeds the 126 MB L2
# DRAM bytes (read+write) per launch of the plane kernels from the ncu captures summarised in profiles/,
# keyed by kernel name -> [(bytes, input elements of the captured launch), ...].  A run takes the capture
# whose size is closest to its own launches and scales it by the input elements (traffic grows in
# proportion to the planes processed; how much of the output is still in the 126 MB L2 when the kernel
# ends differs between a 16-sample and a 256-sample launch, hence two captures).
NCU_TRAFFIC = {
    # profiles/plane_kernels_cfg2_ncu_full.md (batch 16: 4 194 304 input elements) and
    # profiles/plane_kernels_cfg5_dram_bytes.md (batch 256: 67 108 864 input elements)
    "backward_plane_kernel": [(88.25e6, 4194304), (1591.1e6, 67108864)],
    "forward_plane_kernel": [(29.05e6, 4194304), (1281.5e6, 67108864)],
}


def ncu_traffic(kernel, elements):
    """(bytes, text) for a launch over `elements` input elements, or (None, None)."""
    caps = NCU_TRAFFIC.get(kernel)
    if not caps or elements <= 0:
        return None, None
    b, units = min(caps, key=lambda c: abs(np.log(c[1] / elements)))
    text = ("ncu capture of this kernel on a launch of %d input elements (summary under profiles/)%s; "
            "a constant, not measured by this run" % (units, "" if units == elements else ", scaled by the elements per launch"))
    return b * elements / units, text


def describe(name):
    N, C, F, h, w = CONFIGS[name][:5]
    if name == "cfg5":
        return "cfg5: BoxConv2d(%d,%d,%d,%d) fwd+bwd, global batch %d (input %dx%dx%dx%d) divided over the GPUs, fp32, normalize, exact" % (
            C, F, h, w, N, N, C, h, w)
    return "%s: BoxConv2d(%d,%d,%d,%d) fwd+bwd, input %dx%dx%dx%d per GPU, fp32, normalize, exact" % (
        name, C, F, h, w, N, C, h, w)


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
        except Exception:
            pass
    return 6650.0, "fallback (6.65 TB/s; MEASURED_PEAKS.json is absent)"


# ------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's CPU code driven the way its autograd Function
# drives it (box_convolution/box_convolution_function.py:32-65, module.py:216-222)
# ------------------------------------------------------------------------------------------
class CpuReference:
    def __init__(self):
        from oracle import build_ref, oracle
        self.ext = build_ref.load_ref()
        self.kind = "reference" if self.ext is not None else "port"
        self.oracle = oracle
        if self.ext is None:
            oracle.build()
        self.cores = torch.get_num_threads() if self.ext is not None else 1

    def step(self, wl):
        """clip -> de-reparametrize -> integral image -> forward -> backward.  Returns seconds."""
        t0 = time.perf_counter()
        if self.ext is not None:
            x = torch.from_numpy(wl.x)
            go = torch.from_numpy(wl.grad_output)
            stored = [torch.from_numpy(p.copy()) for p in wl.stored]
            self.ext.clip_parameters(*stored, wl.rep_h, wl.rep_w, float(wl.max_h), float(wl.max_w), True)
            actual = [stored[0] * wl.rep_h, stored[1] * wl.rep_h, stored[2] * wl.rep_w, stored[3] * wl.rep_w]
            integ = self.ext.integral_image(x)
            out = self.ext.box_convolution_forward(integ, *actual, True, True)
            self.ext.box_convolution_backward(integ, *actual, go, out, wl.rep_h, wl.rep_w, True, True,
                                              True, True, True, True, True)
        else:
            stored = [p.copy() for p in wl.stored]
            self.oracle.clip_parameters(*stored, wl.rep_h, wl.rep_w, wl.max_h, wl.max_w, True)
            self.oracle.boxconv2d_forward_backward(wl.x, stored, wl.grad_output, wl.rep_h, wl.rep_w, True, True)
        return time.perf_counter() - t0

    def pick_sample(self, name, steps_total, budget_s):
        """Largest batch (<= the config's) whose `steps_total` steps fit in `budget_s`."""
        full_n = CONFIGS[name][0]
        probe = make_workload(name, batch=1)
        self.step(probe)
        per_sample = min(self.step(probe) for _ in range(2))
        n = int(budget_s / max(per_sample * steps_total, 1e-9))
        return max(1, min(full_n, n))


def run_reference(args, rank, world):
    if rank != 0:
        return
    ref = CpuReference()
    n = ref.pick_sample(args.workload, args.steps + args.warmup, 150.0)
    wl = make_workload(args.workload, batch=n)
    for _ in range(args.warmup):
        ref.step(wl)
    times = [ref.step(wl) for _ in range(args.steps)]
    sec = sum(times) / len(times)
    value = wl.outputs / sec / 1e9
    sample = "batch %d of %d of %s per step, %d steps, mean" % (n, CONFIGS[args.workload][0], args.workload, args.steps)
    strong = args.workload == "cfg5"
    config = training_config(args.workload, args.gpus, strong, args.shard_of)
    config.update({
        "l2": "host memory: no device buffers",
        "launch": "host loop over the reference's four extension functions, as its autograd Function calls them",
        "rounds": 1, "round_ms_min": sec * 1e3 * args.steps, "round_ms_max": sec * 1e3 * args.steps,
        "timing": "mean host wall time of `steps` steps on a bounded sample of the batch (see cpu_baseline.sample)",
        "eager_ms_per_step": sec * 1e3, "collective": "none"})
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": ref.cores, "kind": ref.kind, "sample": sample,
                         "os_cpu_count": os.cpu_count()},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# inference workload: the box-block tails of BoxENet on one 512 x 1024 frame
# ------------------------------------------------------------------------------------------
# (count, C = bottleneck channels, F, h, w): BottleneckBoxConv(128,4,h/8,w/8) x8, (64,4,h/4,w/4) x3 and
# (16,2,h/2,w/2) x1 of the reference's BoxENet (examples/Cityscapes/models/ENet.py:61-105), batch 1,
# rounded boxes (exact=False) and BatchNorm/Dropout removed as its runtime script does
# (examples/Cityscapes/convnet-runtime-benchmark.py:38-53): per block ReLU -> BoxConv2d -> + skip -> ReLU.
INFER_LAYERS = [(8, 32, 4, 64, 128), (3, 16, 4, 128, 256), (1, 8, 2, 256, 512)]
INFER_METRIC = "BoxENet box-block tails per 512x1024 frame, batch 1"


def infer_inputs(C, F, h, w, seed, device=None):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((1, C, h, w), generator=g)
    skip = torch.randn((1, C * F, h, w), generator=g)
    return (x.to(device), skip.to(device)) if device is not None else (x, skip)


def infer_module(cls, C, F, h, w, seed):
    import random
    random.seed(seed)                       # reset_parameters draws from Python's generator
    m = cls(C, F, h, w, reparametrization_factor=0.86)
    m.exact = False
    return m


def run_infer(args, rank, world, local_rank):
    """Latency of the box-block tails of one frame: every rank runs the same frame (replicas)."""
    import box_convolution as bc
    from box_convolution import _cabi
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    sampler = ClockSampler(local_rank)
    sampler.start()
    K, W = max(args.steps, 1), max(args.warmup, 3)
    per_layer = []
    launches0 = _cabi.lib.bc_launch_count()
    t_start = time.perf_counter()
    total = {"unfused_eager": 0.0, "fused_eager": 0.0, "fused_graph": 0.0, "fused_graph_cold": 0.0}
    for li, (count, C, F, h, w) in enumerate(INFER_LAYERS):
        m = infer_module(bc.BoxConv2d, C, F, h, w, 100 + li).to(dev).eval()
        # enough distinct (input, skip, output) sets to exceed the 126 MB L2 for the cold figure
        set_bytes = 4 * h * w * (C + 2 * C * F)
        nsets = max(2, int(140e6 // set_bytes) + 1)
        sets = [infer_inputs(C, F, h, w, 1000 * li + i, dev) for i in range(nsets)]

        def unfused(x, skip):
            with torch.no_grad():
                return (skip + m(torch.relu(x))).relu_()

        def fused(x, skip):
            return bc.fused_box_block(m, x, input_relu=True, residual=skip, output_relu=True)

        def timed(fn, rotate):
            for i in range(W):
                fn(*sets[i % nsets if rotate else 0])
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(K):
                fn(*sets[i % nsets if rotate else 0])
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) * 1e3 / K          # us per call

        graphs = [bc.GraphedForward(fused, *sets[i]) for i in range(nsets)]
        it = [0]

        def graph_hot(x, skip):
            return graphs[0].replay()

        def graph_cold(x, skip):
            it[0] += 1
            return graphs[it[0] % nsets].replay()

        r = {"layer": "BoxConv2d(%d,%d,%d,%d)" % (C, F, h, w), "per_frame": count,
             "unfused_eager_us": timed(unfused, True), "fused_eager_us": timed(fused, True),
             "fused_graph_us": timed(graph_hot, False), "fused_graph_cold_us": timed(graph_cold, False)}
        want = unfused(*sets[0])
        err = (fused(*sets[0]) - want).abs().max().item() / max(1.0, want.abs().max().item())
        r["max_rel_err_vs_unfused"] = err
        per_layer.append(r)
        for k in total:
            total[k] += count * r[k + "_us"]
        del graphs, sets
        stage("inference layer %d done" % li)
    # ---- the whole frame as one CUDA graph: the 12 block tails in network order, each with its own
    # module and buffers, the way a deployed network would run them (one graph launch per frame)
    order = [1, 1] + [0] * 8 + [1, 2]           # indices into INFER_LAYERS, BoxENet's order
    frame_sets = []
    for fs in range(2):                         # two frames' worth of buffers (164 MB) for the cold figure
        layers = []
        for pos, li in enumerate(order):
            count, C, F, h, w = INFER_LAYERS[li]
            m = infer_module(bc.BoxConv2d, C, F, h, w, 200 + pos).to(dev).eval()
            layers.append((m,) + infer_inputs(C, F, h, w, 5000 + 100 * fs + pos, dev))
        frame_sets.append(layers)

    def frame(layers):
        outs = []
        for m, x, skip in layers:
            outs.append(bc.fused_box_block(m, x, input_relu=True, residual=skip, output_relu=True))
        return outs

    frame_graphs = []
    for layers in frame_sets:
        for _ in range(3):
            frame(layers)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(g):
            kept = frame(layers)
        frame_graphs.append((g, kept))

    def timed_frames(rotate):
        for i in range(W):
            frame_graphs[i % 2 if rotate else 0][0].replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(K):
            frame_graphs[i % 2 if rotate else 0][0].replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / K

    total["frame_graph"] = timed_frames(False)
    total["frame_graph_cold"] = timed_frames(True)
    stage("frame graphs done")

    t_end = time.perf_counter()
    sampler.stop_flag = True
    sampler.join(timeout=1.0)
    if rank != 0:
        return
    line = {
        "metric": INFER_METRIC, "value": total["frame_graph_cold"], "unit": "us", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": total["frame_graph_cold"] / 1e3, "higher_is_better": False, "scaling": "replicas", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "infer: per block ReLU -> BoxConv2d(exact=False) -> + skip -> ReLU, eval mode, batch 1; "
                               "8 x (32,4,64,128) + 3 x (16,4,128,256) + 1 x (8,2,256,512)",
                   "l2": "value = one CUDA graph per frame (all 12 tails), alternating two frames' buffers (164 MB > L2); "
                         "frame_graph reuses one frame's buffers; the per-layer figures are one graph launch per layer"},
        "totals_us": total, "layers": per_layer,
        "gpu_launches": int(_cabi.lib.bc_launch_count() - launches0),
        "clocks": sampler.summary(t_start, t_end),
    }
    print(json.dumps(line), flush=True)


def run_infer_reference(args, rank, world):
    """The same block tails through the reference's CPU extension, driven as its autograd Function
    drives it (integral_image -> box_convolution_forward), all host threads torch gives it."""
    if rank != 0:
        return
    from oracle import build_ref, oracle
    ext = build_ref.load_ref()
    kind = "reference" if ext is not None else "port"
    sys.path.insert(0, os.path.join(ROOT, "box-convolutions_b200"))
    import random
    total, per_layer = 0.0, []
    reps = max(1, min(args.steps, 3))
    for li, (count, C, F, h, w) in enumerate(INFER_LAYERS):
        # same boxes as our arm: the reference's own initialisation rule, seeded alike
        from box_convolution.module import BoxConv2d
        m = infer_module(BoxConv2d, C, F, h, w, 100 + li)
        pix = [p.detach() * f for p, f in zip((m.x_min, m.x_max, m.y_min, m.y_max),
                                              (m.reparametrization_h, m.reparametrization_h,
                                               m.reparametrization_w, m.reparametrization_w))]
        x, skip = infer_inputs(C, F, h, w, 1000 * li)

        def block():
            xr = torch.relu(x)
            if ext is not None:
                out = ext.box_convolution_forward(ext.integral_image(xr), *pix, True, False)
            else:
                integ = oracle.integral_image(xr.numpy())
                out = torch.from_numpy(oracle.box_convolution_forward(integ, *[p.numpy() for p in pix], True, False))
            return (skip + out.view_as(skip)).relu_()

        block()
        t0 = time.perf_counter()
        for _ in range(reps):
            block()
        us = (time.perf_counter() - t0) / reps * 1e6
        per_layer.append({"layer": "BoxConv2d(%d,%d,%d,%d)" % (C, F, h, w), "per_frame": count, "us": us})
        total += count * us
    cores = torch.get_num_threads() if ext is not None else 1
    line = {
        "impl": "reference", "metric": INFER_METRIC, "value": total, "unit": "us", "n_gpus": args.gpus,
        "steps": reps, "warmup": 1, "ms_per_step": total / 1e3, "higher_is_better": False, "scaling": "replicas",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "infer (see the main arm)", "host_threads": cores, "os_cpu_count": os.cpu_count()},
        "layers": per_layer,
        "cpu_baseline": {"value": total, "unit": "us", "cores": cores, "kind": kind,
                         "sample": "each of the three layer shapes timed %d times, scaled by its count per frame" % reps},
        "e2e": {"value": total, "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------
class ClockSampler(threading.Thread):
    """Polls NVML (read-only) for SM clock and throttle reasons of one GPU."""
    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
        0x4: "sw_power_cap", 0x80: "hw_power_brake", 0x2: "applications_clocks_setting",
    }

    def __init__(self, index, active=True, period_s=0.02):
        super().__init__(daemon=True)
        self.samples = []      # (time, sm_mhz, reasons_bitmask, power_w)
        self.stop_flag = False
        self.active = active   # NVML is only called while this is set (its calls contend with kernel launches)
        self.period_s = period_s
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.max_mhz = None

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        while not self.stop_flag:
            if not self.active:
                time.sleep(self.period_s)
                continue
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                try:
                    rs = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    rs = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                pw = nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0
                self.samples.append((time.perf_counter(), mhz, rs, pw))
            except Exception:
                pass
            time.sleep(self.period_s)

    def summary(self, t0, t1):
        sel = [s for s in self.samples if t0 <= s[0] <= t1]
        if not sel:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        mask = 0
        for s in sel:
            mask |= s[2]
        return {
            "sm_mhz": statistics.median(s[1] for s in sel), "sm_max_mhz": self.max_mhz,
            "reasons": sorted(n for b, n in self.REASONS.items() if mask & b),
            "samples": len(sel), "power_w_max": max(s[3] for s in sel),
        }


# ------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------
def kernel_algorithmic_bytes(kernel, N, C, F, h, w):
    E, Ei = N * C * h * w, N * C * (h + 1) * (w + 1)
    return {
        # two launches per step on the large-plane path (input planes, then F times as many grad_output
        # planes): mean bytes per launch
        "integral_image_kernel": 4 * (1 + F) * (E + Ei) // 2,
        "forward_global_kernel": 4 * (Ei + F * E),
        "backward_global_kernel": 4 * (F * Ei + 2 * E),
        "forward_band_kernel": 4 * (Ei + F * E),
        "backward_band_kernel": 4 * (F * Ei + 2 * E),
        "forward_plane_kernel": 4 * E * (1 + F),
        "backward_plane_kernel": 4 * E * (F + 2),
    }.get(kernel)


def run_integral(args, rank, world, local_rank):
    """cfg4: the integral image alone, 1024 planes of 512 x 1024 U[0,1) per GPU."""
    import box_convolution as bc
    from box_convolution import _cabi
    from workloads import make_integral_workload

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    planes, h, w = 1024, 512, 1024
    gen = torch.Generator(device=dev)
    gen.manual_seed(1004 + rank)
    x = torch.rand((planes, h, w), device=dev, generator=gen)
    out = torch.empty((planes, h + 1, w + 1), device=dev)
    stream = torch.cuda.current_stream().cuda_stream

    def step():
        _cabi.check(_cabi.lib.bc_integral_image(x.data_ptr(), out.data_ptr(), planes, h, w, stream), "integral_image")

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / args.steps
    alg = 4 * planes * (h * w + (h + 1) * (w + 1))
    peak, peak_src = measured_peak()
    achieved = alg / (ms * 1e-3) / 1e9
    cpu_baseline = None
    if rank == 0 and not args.skip_cpu_baseline:
        ref = CpuReference()
        sample = make_integral_workload(planes=64, h=h, w=w)
        t = torch.from_numpy(sample)
        fn = (lambda: ref.ext.integral_image(t)) if ref.ext is not None else (lambda: ref.oracle.integral_image(sample))
        fn()
        t0 = time.perf_counter()
        for _ in range(5):
            fn()
        sec = (time.perf_counter() - t0) / 5
        cpu_baseline = {"value": 4 * 64 * (h * w + (h + 1) * (w + 1)) / sec / 1e9, "unit": "GB/s", "cores": ref.cores,
                        "kind": ref.kind, "sample": "64 of 1024 planes, 1 warm-up + 5 runs, mean %.3f s" % sec}
    if rank == 0:
        print(json.dumps({
            "metric": "integral_image algorithmic HBM GB/s", "value": achieved * world, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "cfg4: integral image of 1024 planes of 512x1024 per GPU, U[0,1)",
                       "l2": "4.3 GB touched per launch"},
            "roofline": {"bound": "hbm", "kernel": "integral_image_kernel", "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak,
                         # ncu capture of the integral image kernel on cfg4 (summary under profiles/): 2.148 GB read + 2.108 GB written
                         "traffic": 4.2556e9, "algorithmic_bytes": alg,
                         "mean_us": ms * 1e3, "peak_source": peak_src},
            "cpu_baseline": cpu_baseline, "gpu_launches": args.steps}), flush=True)


class TrainingRun:
    """One workload on this rank: module, rotating buffer sets, one CUDA graph per buffer set holding
    the compute of a step (clip, forward, backward, finishing kernel)."""

    def __init__(self, args, name, rank, world, dev):
        import box_convolution as bc
        from box_convolution import _cabi
        self.bc, self.cabi = bc, _cabi
        self.args, self.name, self.rank, self.world, self.dev = args, name, rank, world, dev
        # cfg5 is the batch-sharded configuration: a global batch of 256 divided over the ranks (strong
        # scaling); every other workload is run once per rank (weak scaling)
        self.strong = name == "cfg5"
        full_n = CONFIGS[name][0]
        if self.strong and full_n % world:
            raise SystemExit("cfg5: the global batch of %d does not divide over %d GPUs" % (full_n, world))
        # the host copy of the workload feeds buffer set 0 of rank 0, the end-to-end leg and the CPU baseline
        shards = world * max(1, getattr(args, "shard_of", 1) // world) if self.strong else 1
        if self.strong and full_n % shards:
            raise SystemExit("cfg5: the global batch of %d does not divide into %d shards" % (full_n, shards))
        self.wl = wl = make_workload(name, batch=full_n // shards if self.strong else None)
        N, C, F, h, w = wl.shape
        self.module = m = bc.BoxConv2d(C, F, wl.max_h, wl.max_w, reparametrization_factor=8, normalize=True).to(dev)
        with torch.no_grad():
            for p, v in zip((m.x_min, m.x_max, m.y_min, m.y_max), wl.stored):
                p.copy_(torch.from_numpy(v))
        m.train()
        self.params = [m.x_min, m.x_max, m.y_min, m.y_max]
        # distinct inputs per rank and per buffer set (same distribution)
        gen = torch.Generator(device=dev)
        gen.manual_seed(1234 + rank)
        self.xs, self.gos = [], []
        for s in range(BUFFER_SETS):
            if s == 0 and rank == 0:
                self.xs.append(torch.from_numpy(wl.x).to(dev).requires_grad_())
                self.gos.append(torch.from_numpy(wl.grad_output).to(dev))
            else:
                self.xs.append(torch.randn((N, C, h, w), device=dev, generator=gen).requires_grad_())
                self.gos.append(torch.randn((N, C * F, h, w), device=dev, generator=gen))
        self.graphs, self.outs, self.packed = None, [], []
        self.works = [None] * BUFFER_SETS
        self.step_index = 0

    def compute(self, s):
        for p in self.params:
            p.grad = None
        self.xs[s].grad = None
        out = self.module(self.xs[s])
        out.backward(self.gos[s])
        return out

    def eager_step(self, s):
        out = self.compute(s)
        if self.world > 1:
            self.bc.allreduce_box_gradients(self.module)
        return out

    def warm_up_and_capture(self):
        import torch.distributed as dist
        for i in range(max(self.args.warmup, 3)):
            self.eager_step(i % BUFFER_SETS)
        torch.cuda.synchronize()
        before = self.cabi.lib.bc_launch_count()
        self.compute(0)
        self.launches_per_step = self.cabi.lib.bc_launch_count() - before
        torch.cuda.synchronize()
        if self.args.no_graph:
            return
        self.graphs, pool = [], None
        for s in range(BUFFER_SETS):
            g = torch.cuda.CUDAGraph()
            for p in self.params:
                p.grad = None
            self.xs[s].grad = None
            with torch.cuda.graph(g, pool=pool):
                self.outs.append(self.compute(s))
                self.packed.append(self.bc.packed_box_gradient(self.module)[0])
            pool = g.pool()
            self.graphs.append(g)
        for g in self.graphs:
            g.replay()
        torch.cuda.synchronize()
        if self.world > 1:
            for s in range(BUFFER_SETS):        # the communicator's first collectives, outside any timing
                dist.all_reduce(self.packed[s])
            torch.cuda.synchronize()

    def run_steps(self, k):
        """k consecutive steps, the same way at every GPU count: one graph replay per step; with more than
        one GPU the all-reduce of the step's packed gradient is issued right behind it (asynchronously:
        it runs on the process group's own stream, under the kernels of the next step).  A buffer set is
        not replayed again before its previous reduction has finished (a stream-side wait)."""
        import torch.distributed as dist
        for _ in range(k):
            s = self.step_index % BUFFER_SETS
            self.step_index += 1
            if self.graphs is None:
                self.eager_step(s)
                continue
            if self.works[s] is not None:
                self.works[s].wait()
                self.works[s] = None
            self.graphs[s].replay()
            if self.world > 1:
                self.works[s] = dist.all_reduce(self.packed[s], async_op=True)

    def replay_only_ms_per_step(self, rounds=8):
        """The same graph replays without the all-reduce behind them (median of a few rounds, max over
        ranks): what the step costs before any communication is added."""
        import torch.distributed as dist
        if self.graphs is None:
            return None
        K = self.args.steps
        self.drain()
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier()
        events = [torch.cuda.Event(enable_timing=True) for _ in range(rounds + 1)]
        events[0].record()
        for r in range(rounds):
            for i in range(K):
                self.graphs[i % BUFFER_SETS].replay()
            events[r + 1].record()
        torch.cuda.synchronize()
        t = torch.tensor([events[r].elapsed_time(events[r + 1]) for r in range(rounds)], device=self.dev, dtype=torch.float64)
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return statistics.median(t.tolist()) / K

    def drain(self):
        for s in range(BUFFER_SETS):
            if self.works[s] is not None:
                self.works[s].wait()
                self.works[s] = None

    def timed_rounds(self, sampler):
        """R consecutive rounds of K steps, one CUDA event between rounds; returns the per-round times
        (ms, max over ranks) and the host-clock window of the timed region."""
        import torch.distributed as dist
        K = self.args.steps
        self.run_steps(max(self.args.warmup, 3))
        self.drain()
        torch.cuda.synchronize()
        # pilot round: how many rounds make the timed region long enough for clock sampling
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record()
        self.run_steps(K)
        self.drain()
        p1.record()
        torch.cuda.synchronize()
        pilot = torch.tensor([p0.elapsed_time(p1)], device=self.dev, dtype=torch.float64)
        if self.world > 1:
            dist.all_reduce(pilot, op=dist.ReduceOp.MAX)
        rounds = self.args.rounds or int(min(1000, max(15, -(-self.args.min_timed_ms // max(float(pilot.item()), 1e-3)))))
        events = [torch.cuda.Event(enable_timing=True) for _ in range(rounds + 1)]
        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        if sampler is not None:
            sampler.active = True
        t_start = time.perf_counter()
        events[0].record()
        for r in range(rounds):
            self.run_steps(K)
            if r == rounds - 1:
                self.drain()                    # the region ends when the last reduction has finished
            events[r + 1].record()
        torch.cuda.synchronize()
        t_end = time.perf_counter()
        if sampler is not None:
            sampler.active = False
        if self.world > 1:
            dist.barrier()
        per_round = torch.tensor([events[r].elapsed_time(events[r + 1]) for r in range(rounds)],
                                 device=self.dev, dtype=torch.float64)
        if self.world > 1:
            dist.all_reduce(per_round, op=dist.ReduceOp.MAX)
        return per_round.tolist(), (t_start, t_end)

    def per_kernel(self):
        """Device time of every kernel of the step, from the library's own event pairs around each
        launch, over an eager repeat of K steps (events cannot be read back from a replayed graph)."""
        import ctypes
        lib, K = self.cabi.lib, self.args.steps
        self.cabi.check(lib.bc_profile_start(K * max(self.launches_per_step, 1) + 16), "bc_profile_start")
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(K):
            self.eager_step(i % BUFFER_SETS)
        e1.record()
        torch.cuda.synchronize()
        lib.bc_profile_stop()
        eager_ms = e0.elapsed_time(e1) / K
        per = {}
        kid, ms = ctypes.c_int(), ctypes.c_float()
        for i in range(lib.bc_profile_count()):
            self.cabi.check(lib.bc_profile_get(i, ctypes.byref(kid), ctypes.byref(ms)), "bc_profile_get")
            per.setdefault(lib.bc_kernel_name(kid.value).decode(), []).append(ms.value)
        kernels = {k: {"launches": len(v), "mean_us": 1e3 * sum(v) / len(v), "total_ms": sum(v)} for k, v in per.items()}
        roofline = None
        if kernels:
            N, C, F, h, w = self.wl.shape
            top = max(kernels, key=lambda k: kernels[k]["total_ms"])
            alg = kernel_algorithmic_bytes(top, N, C, F, h, w)
            peak, peak_src = measured_peak()
            if alg is not None:
                achieved = alg / (kernels[top]["mean_us"] * 1e-6) / 1e9
                traffic, traffic_source = ncu_traffic(top, N * C * h * w)
                roofline = {"bound": "hbm", "kernel": top, "achieved": achieved, "peak": peak, "unit": "GB/s",
                            "frac": achieved / peak, "traffic": traffic, "traffic_source": traffic_source,
                            "algorithmic_bytes": alg, "mean_us": kernels[top]["mean_us"], "peak_source": peak_src,
                            "kernels": {k: round(v["mean_us"], 2) for k, v in kernels.items()}}
        return roofline, eager_ms

    def check_sharding(self):
        """On more than one GPU, outside any timing: (1) the all-reduced packed gradient of every buffer
        set equals the sum of the ranks' local gradients; (2) rank 0 recomputes the whole global batch of
        buffer set 0 from the ranks' inputs and compares every rank's output and grad-input shard with its
        slice, and the reduced parameter gradient with the full-batch one."""
        import torch.distributed as dist
        world, rank, dev = self.world, self.rank, self.dev
        self.drain()
        torch.cuda.synchronize()
        worst = {"allreduce_vs_sum_of_locals": 0.0, "output_shard_vs_full_batch": 0.0,
                 "grad_input_shard_vs_full_batch": 0.0, "reduced_grad_vs_full_batch": 0.0}

        def rel(a, b):
            return float((a.double() - b.double()).abs().max() / b.double().abs().max().clamp_min(1e-30))

        local0 = None
        for s in range(BUFFER_SETS):
            if self.graphs is not None:
                self.graphs[s].replay()
                packed = self.packed[s]
            else:
                self.compute(s)
                packed = self.bc.packed_box_gradient(self.module)[0]
            local = packed.clone()
            gathered = [torch.empty_like(local) for _ in range(world)]
            dist.all_gather(gathered, local)
            dist.all_reduce(packed)
            want = torch.stack(gathered).double().sum(0)
            worst["allreduce_vs_sum_of_locals"] = max(worst["allreduce_vs_sum_of_locals"], rel(packed, want))
            if s == 0:
                local0 = (packed.clone(), self.outs[0].detach().clone() if self.graphs is not None else None,
                          self.xs[0].grad.detach().clone())
        # (2) the global batch on rank 0
        N, C, F, h, w = self.wl.shape
        reduced, out_shard, gin_shard = local0
        if out_shard is None:
            out_shard = self.compute(0).detach().clone()
            gin_shard = self.xs[0].grad.detach().clone()

        def gather_all(t):
            full = torch.empty((world * t.shape[0],) + tuple(t.shape[1:]), device=dev, dtype=t.dtype)
            dist.all_gather_into_tensor(full, t.contiguous())
            return full

        x_all, go_all = gather_all(self.xs[0].detach()), gather_all(self.gos[0])
        out_all, gin_all = gather_all(out_shard), gather_all(gin_shard)
        if rank == 0:
            x_all.requires_grad_()
            for p in self.params:
                p.grad = None
            out_full = self.module(x_all)
            out_full.backward(go_all)
            full_grad = self.bc.packed_box_gradient(self.module)[0]
            worst["output_shard_vs_full_batch"] = rel(out_all, out_full.detach())
            worst["grad_input_shard_vs_full_batch"] = rel(gin_all, x_all.grad)
            worst["reduced_grad_vs_full_batch"] = rel(reduced, full_grad)
        verdict = torch.tensor([worst[k] for k in sorted(worst)], device=dev, dtype=torch.float64)
        dist.all_reduce(verdict, op=dist.ReduceOp.MAX)
        worst = dict(zip(sorted(worst), verdict.tolist()))
        # sums of identical terms in another order: 1e-5; shards are computed plane by plane by the same
        # kernels: 1e-6 (expected exactly 0); full-batch gradient against the sum of shard gradients: 1e-3
        limits = {"allreduce_vs_sum_of_locals": 1e-5, "output_shard_vs_full_batch": 1e-6,
                  "grad_input_shard_vs_full_batch": 1e-6, "reduced_grad_vs_full_batch": 1e-3}
        ok = all(worst[k] <= limits[k] for k in worst)
        del x_all, go_all, out_all, gin_all
        torch.cuda.empty_cache()
        return ("ok" if ok else "FAILED"), worst

    def end_to_end(self):
        """The same step from pinned host buffers to host results through HostPipeline, and the bare
        bidirectional copies of the same bytes as a floor."""
        import torch.distributed as dist
        args, wl, dev, world = self.args, self.wl, self.dev, self.world
        N, C, F, h, w = wl.shape
        hx = torch.from_numpy(wl.x).pin_memory()
        hgo = torch.from_numpy(wl.grad_output).pin_memory()
        depth = max(1, args.e2e_depth)
        results = [(torch.empty((N, C * F, h, w), dtype=torch.float32).pin_memory(),
                    torch.empty((N, C, h, w), dtype=torch.float32).pin_memory(),
                    torch.empty((4, C, F), dtype=torch.float32).pin_memory()) for _ in range(depth)]
        hout, hgin, hgp = results[0]
        pipe = self.bc.HostPipeline(self.module, N, h, w, chunks=args.e2e_chunks, depth=depth)
        k_e2e = max(3, min(args.steps, 20))
        for _ in range(2):
            pipe.step(hx, hgo, hout, hgin, hgp)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        w0 = time.perf_counter()
        tickets = []
        for i in range(k_e2e):
            if i >= depth:
                pipe.wait(tickets[i - depth])           # results of batch i-depth are on the host
            tickets.append(pipe.submit(hx, hgo, *results[i % depth]))
        for t in tickets[-depth:]:
            pipe.wait(t)
        torch.cuda.synchronize()
        sec = (time.perf_counter() - w0) / k_e2e
        # floor: the same bytes as plain asynchronous copies, both directions at once, nothing else
        up, down = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        dx, dgo = torch.empty_like(hx, device=dev), torch.empty_like(hgo, device=dev)
        dout, dgin = torch.empty_like(hout, device=dev), torch.empty_like(hgin, device=dev)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        f0 = time.perf_counter()
        for _ in range(k_e2e):
            with torch.cuda.stream(up):
                dx.copy_(hx, non_blocking=True)
                dgo.copy_(hgo, non_blocking=True)
            with torch.cuda.stream(down):
                hout.copy_(dout, non_blocking=True)
                hgin.copy_(dgin, non_blocking=True)
        torch.cuda.synchronize()
        floor = (time.perf_counter() - f0) / k_e2e
        if world > 1:
            t = torch.tensor([sec, floor], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            sec, floor = (float(v) for v in t.tolist())
        return {"value": wl.outputs * world / sec / 1e9, "unit": UNIT,
                "h2d_bytes_per_step": hx.numel() * 4 + hgo.numel() * 4,
                "d2h_bytes_per_step": (hout.numel() + hgin.numel() + hgp.numel()) * 4,
                "ms_per_step": sec * 1e3, "copy_floor_ms": floor * 1e3, "steps": k_e2e, "chunks": args.e2e_chunks,
                "batches_in_flight": depth,
                "api": "box_convolution.HostPipeline.submit/wait -> bc_boxconv2d_host_step (C ABI, pinned host buffers in and out, "
                       "chunked copy/compute overlap on 3 streams; every batch's inputs go up and its results come back inside the "
                       "timed region); copy_floor_ms = the same bytes as bare cudaMemcpyAsync in both directions at once, "
                       "per rank, max over ranks"}

    def release(self):
        self.graphs, self.outs, self.packed, self.xs, self.gos = None, [], [], [], []
        torch.cuda.empty_cache()


def training_config(name, world, strong, shard_of=1):
    """The keys of `config` that both arms print alike."""
    full_n = CONFIGS[name][0]
    per_gpu = full_n // (world * max(1, shard_of // world)) if strong else full_n
    return {"workload": describe(name), "global_batch": per_gpu * world, "batch_per_gpu": per_gpu}


def summarise_rounds(per_round, K, outputs_per_step):
    med = statistics.median(per_round)
    return {"ms_per_step": med / K, "value": outputs_per_step / (med / K * 1e-3) / 1e9,
            "rounds": len(per_round), "round_ms_median": med, "round_ms_min": min(per_round),
            "round_ms_max": max(per_round)}


def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    stage("process group ready (world %d)" % world)
    # NVML is polled by rank 0 only, and only while a timed region is running
    sampler = ClockSampler(local_rank, active=False) if rank == 0 else None
    if sampler is not None:
        sampler.start()

    run = TrainingRun(args, args.workload, rank, world, dev)
    wl = run.wl
    N, C, F, h, w = wl.shape
    stage("eager warm-up and graph capture")
    run.warm_up_and_capture()
    stage("timed region: rounds of %d steps" % args.steps)
    per_round, (t_start, t_end) = run.timed_rounds(sampler)
    main = summarise_rounds(per_round, args.steps, wl.outputs * world)
    replay_only = run.replay_only_ms_per_step() if world > 1 else None
    stage("eager repeat with per-kernel events")
    roofline, eager_ms = run.per_kernel()

    sharding = None
    if world > 1:
        stage("sharding check")
        sharding = run.check_sharding()

    e2e = None
    if not args.skip_e2e:
        stage("end-to-end leg")
        e2e = run.end_to_end()

    clocks = sampler.summary(t_start, t_end) if sampler is not None else None

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.skip_cpu_baseline:
        stage("cpu baseline")
        ref = CpuReference()
        n = ref.pick_sample(args.workload, 6, 20.0)
        sample_wl = make_workload(args.workload, batch=n)
        ref.step(sample_wl)
        times = [ref.step(sample_wl) for _ in range(5)]
        sec = sum(times) / len(times)
        cpu_baseline = {"value": sample_wl.outputs / sec / 1e9, "unit": UNIT, "cores": ref.cores,
                        "kind": ref.kind, "os_cpu_count": os.cpu_count(),
                        "sample": "batch %d of %d of %s, 1 warm-up + 5 steps, mean %.3f s per step" % (
                            n, N, args.workload, sec)}

    launches_per_step = run.launches_per_step
    launch_text = ("eager" if run.graphs is None else
                   "one cuda graph replay (clip+forward+backward) per step at every GPU count, %d buffer sets in turn%s" % (
                       BUFFER_SETS, "; the step's all-reduce is issued asynchronously behind its replay and overlaps the next step"
                       if world > 1 else ""))
    run.release()

    # the 1/8-frame block at batch 16 per GPU (the cfg2 workload) as an extra key of the same line
    extra = None
    if args.workload == "cfg5" and not args.skip_cfg2:
        stage("cfg2 (batch 16 per GPU) for the extra key")
        small = TrainingRun(args, "cfg2", rank, world, dev)
        small.warm_up_and_capture()
        rounds2, _ = small.timed_rounds(None)
        extra = summarise_rounds(rounds2, args.steps, small.wl.outputs * world)
        extra["roofline"], extra["eager_ms_per_step"] = small.per_kernel()
        extra["hbm_gbs_step"] = small.wl.algorithmic_bytes * world / (extra["ms_per_step"] * 1e-3) / 1e9
        extra["config"] = dict(training_config("cfg2", world, False), scaling="weak")
        small.release()

    if sampler is not None:
        sampler.stop_flag = True
        sampler.join(timeout=1.0)

    failed = sharding is not None and sharding[0] != "ok"
    if rank == 0:
        config = training_config(args.workload, world, run.strong, args.shard_of)
        config.update({
            "l2": "rotating %d input/output buffer sets (%.0f MB touched per set)" % (BUFFER_SETS, wl.algorithmic_bytes / 1e6),
            "launch": launch_text,
            "rounds": main["rounds"], "round_ms_min": main["round_ms_min"], "round_ms_max": main["round_ms_max"],
            "timing": "value = median over `rounds` consecutive rounds of `steps` steps, one CUDA event between rounds, "
                      "max over ranks per round; barrier + synchronize before the first and after the last round",
            "eager_ms_per_step": eager_ms,
            "collective": "nccl all_reduce of the packed (4,C,F) parameter gradient" if world > 1 else "none"})
        line = {
            "metric": METRIC, "value": main["value"], "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": main["ms_per_step"], "higher_is_better": True,
            "scaling": "strong" if run.strong else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config,
            "hbm_gbs_step": wl.algorithmic_bytes * world / (main["ms_per_step"] * 1e-3) / 1e9,
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
            "gpu_launches": int(launches_per_step * args.steps * main["rounds"]), "clocks": clocks,
        }
        if replay_only is not None:
            line["breakdown"] = {"replay_only_ms_per_step": replay_only, "with_allreduce_ms_per_step": main["ms_per_step"],
                                 "note": "the same graph replays timed without and with the per-step all-reduce"}
        if sharding is not None:
            line["allreduce_check"] = sharding[0]
            line["allreduce_check_max_rel_err"] = sharding[1]
        if extra is not None:
            line["cfg2"] = extra
        print(json.dumps(line), flush=True)
    stage("done")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if failed:
        raise SystemExit("bench: the sharded results do not match the full batch: %r" % (sharding[1],))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", default="cfg5", choices=sorted(CONFIGS) + ["cfg4", "infer"])
    ap.add_argument("--rounds", type=int, default=0, help="timed rounds of --steps steps (0: at least 15, more until --min-timed-ms)")
    ap.add_argument("--min-timed-ms", type=float, default=300.0, help="shortest timed region when --rounds is 0")
    ap.add_argument("--skip-cfg2", action="store_true", help="cfg5 only: leave out the extra cfg2 key")
    ap.add_argument("--shard-of", type=int, default=1,
                    help="cfg5 only: give every rank the shard it would have in a job of this many GPUs (e.g. "
                         "`--gpus 1 --shard-of 8` times one GPU's share of the 8-GPU job, without the collective)")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-cpu-baseline", action="store_true")
    ap.add_argument("--e2e-chunks", type=int, default=8)
    ap.add_argument("--e2e-depth", type=int, default=2, help="batches in flight in the end-to-end leg")
    ap.add_argument("--max-seconds", type=int, default=600, help="host-side watchdog for the whole run")
    args = ap.parse_args()
    arm_watchdog(args.max_seconds)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("launch with: python -m torch.distributed.run --nproc-per-node %d bench.py --gpus %d ..."
                         % (args.gpus, args.gpus))
    if args.impl == "reference":
        if args.workload == "cfg4":
            raise SystemExit("--impl reference supports the BoxConv2d workloads; cfg4 prints its CPU baseline in the main line")
        if args.workload == "infer":
            run_infer_reference(args, rank, world)
        else:
            run_reference(args, rank, world)
    else:
        if not torch.cuda.is_available():
            raise SystemExit("bench.py --impl ours needs a GPU: the CUDA library has no CPU fallback")
        if args.workload == "cfg4":
            run_integral(args, rank, world, local_rank)
        elif args.workload == "infer":
            run_infer(args, rank, world, local_rank)
        else:
            run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
