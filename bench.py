#!/usr/bin/env python
"""Benchmark of the BoxConv2d forward+backward hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg2]

(`--workload cfg4` times the integral image alone, `--workload infer` the batch-1 inference block
tails of one frame; the default and the contract line are cfg2.)

One step = one training pass of the box block over one batch of synthetic input: parameter
clip, forward, backward (grad-input and the four parameter gradients) and, on more than one GPU,
the all-reduce of the packed (4, C, F) parameter gradient.  Each rank works on its own batch of
the per-GPU shape (weak scaling); `value` is the whole job's output elements per second.

The line printed by rank 0 carries, besides the contract keys:
  roofline      achieved HBM GB/s of the dominant kernel (algorithmic bytes / mean device time of
                that kernel, from per-kernel CUDA events recorded by the library during an eager
                repeat of the timed steps) against the measured copy bandwidth of this pool
  cpu_baseline  the reference's own CPU code on this machine's host cores (N=1 only)
  e2e           the same metric from pinned host buffers to host results through the module
  clocks        SM clock and throttle reasons sampled through NVML while the GPU was busy

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
# DRAM bytes (read+write) per launch of the dominant kernel from the ncu capture summarised in
# profiles/, keyed by kernel name -> (bytes, units it was captured on); scaled by units at run time.
NCU_TRAFFIC = {
    # ncu capture of the plane kernels on cfg2 (summary under profiles/): 83.93 MB read + 4.00 MB written on cfg2 (4 194 304 input
    # elements); below the 100.7 MB algorithmic figure because the 126 MB L2 still holds part of the
    # 16.8 MB grad_input when the kernel ends
    "backward_plane_kernel": (87.93e6, 4194304),
    "forward_plane_kernel": (25.81e6, 4194304),
}


def describe(name):
    N, C, F, h, w = CONFIGS[name][:5]
    return "%s: BoxConv2d(%d,%d,%d,%d) fwd+bwd, input %dx%dx%dx%d per GPU, fp32, normalize, exact" % (
        name, C, F, h, w, N, C, h, w)


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
        except Exception:
            pass
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


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
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": describe(args.workload), "host_threads": ref.cores,
                   "os_cpu_count": os.cpu_count()},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": ref.cores, "kind": ref.kind, "sample": sample},
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

    def __init__(self, index):
        super().__init__(daemon=True)
        self.samples = []      # (time, sm_mhz, reasons_bitmask, power_w)
        self.stop_flag = False
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
            time.sleep(0.002)

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


def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist
    import box_convolution as bc
    from box_convolution import _cabi

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    stage("process group ready (world %d)" % world)
    sampler = ClockSampler(local_rank)
    sampler.start()

    # cfg5 is the batch-sharded configuration: a global batch of 256 divided over the ranks (strong
    # scaling); every other workload is run once per rank (weak scaling)
    strong = args.workload == "cfg5"
    wl = make_workload(args.workload, batch=CONFIGS[args.workload][0] // world if strong else None)
    N, C, F, h, w = wl.shape
    module = bc.BoxConv2d(C, F, wl.max_h, wl.max_w, reparametrization_factor=8, normalize=True).to(dev)
    with torch.no_grad():
        for p, v in zip((module.x_min, module.x_max, module.y_min, module.y_max), wl.stored):
            p.copy_(torch.from_numpy(v))
    module.train()
    params = [module.x_min, module.x_max, module.y_min, module.y_max]

    # distinct inputs per rank and per buffer set (same distribution)
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234 + rank)
    xs, gos = [], []
    for s in range(BUFFER_SETS):
        if s == 0 and rank == 0:
            xs.append(torch.from_numpy(wl.x).to(dev).requires_grad_())
            gos.append(torch.from_numpy(wl.grad_output).to(dev))
        else:
            xs.append(torch.randn((N, C, h, w), device=dev, generator=gen).requires_grad_())
            gos.append(torch.randn((N, C * F, h, w), device=dev, generator=gen))

    def compute(s):
        for p in params:
            p.grad = None
        xs[s].grad = None
        out = module(xs[s])
        out.backward(gos[s])
        return out

    def step(s):
        out = compute(s)
        if world > 1:
            bc.allreduce_box_gradients(module)
        return out

    stage("eager warm-up")
    # ---- warm-up (eager), then capture one CUDA graph per buffer set
    for i in range(max(args.warmup, 3)):
        step(i % BUFFER_SETS)
    torch.cuda.synchronize()
    launches_before = _cabi.lib.bc_launch_count()
    step(0)
    launches_per_step = _cabi.lib.bc_launch_count() - launches_before
    torch.cuda.synchronize()

    # The graphs hold the compute of a step (clip, forward, backward); the all-reduce of the packed
    # parameter gradient is issued after each replay on the same stream, outside the graph.
    graphs, packed, multi = None, [], None
    if not args.no_graph:
        stage("capturing %d CUDA graphs" % BUFFER_SETS)
        graphs, keep = [], []
        pool = None
        for s in range(BUFFER_SETS):
            g = torch.cuda.CUDAGraph()
            for p in params:
                p.grad = None
            xs[s].grad = None
            with torch.cuda.graph(g, pool=pool):
                keep.append(compute(s))
                packed.append(bc.packed_box_gradient(module)[0])
            pool = g.pool()
            graphs.append(g)
        for s in range(BUFFER_SETS):
            graphs[s].replay()
        torch.cuda.synchronize()
        if world == 1:
            # one more graph that runs a step on every buffer set in turn: BUFFER_SETS steps per launch
            multi = torch.cuda.CUDAGraph()
            for p in params:
                p.grad = None
            with torch.cuda.graph(multi, pool=pool):
                for s in range(BUFFER_SETS):
                    keep.append(compute(s))
            multi.replay()
            torch.cuda.synchronize()

    # With graphs, the all-reduce of step k runs on a side stream while step k+1 computes (the way a
    # trainer overlaps gradient reduction with the rest of the backward pass); a buffer set is not
    # reused before its reduction has finished, and the timed region ends only when all are done.
    comm_stream = torch.cuda.Stream(dev) if world > 1 else None
    reduced = [None] * BUFFER_SETS

    def run_steps(k):
        main = torch.cuda.current_stream()
        done = 0
        if multi is not None:
            for _ in range(k // BUFFER_SETS):
                multi.replay()
            done = (k // BUFFER_SETS) * BUFFER_SETS
        for i in range(done, k):
            s = i % BUFFER_SETS
            if graphs is not None:
                if reduced[s] is not None:
                    main.wait_event(reduced[s])
                graphs[s].replay()
                if world > 1:
                    ready = torch.cuda.Event()
                    ready.record(main)
                    with torch.cuda.stream(comm_stream):
                        comm_stream.wait_event(ready)
                        dist.all_reduce(packed[s])
                        reduced[s] = torch.cuda.Event()
                        reduced[s].record(comm_stream)
            else:
                step(s)
        if comm_stream is not None:
            main.wait_stream(comm_stream)

    # ---- the timed region
    stage("timed region: %d steps" % args.steps)
    run_steps(max(args.warmup, 3))
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start = time.perf_counter()
    ev0.record()
    run_steps(args.steps)
    ev1.record()
    torch.cuda.synchronize()
    t_end = time.perf_counter()
    if world > 1:
        dist.barrier()
    ms_total = ev0.elapsed_time(ev1)
    if world > 1:
        t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_per_step = ms_total / args.steps
    value = wl.outputs * world / (ms_per_step * 1e-3) / 1e9

    stage("eager repeat with per-kernel events")
    # ---- per-kernel device times: the same steps, eagerly, with the library's event pairs
    roofline = None
    eager_ms = None
    _cabi.check(_cabi.lib.bc_profile_start(args.steps * max(launches_per_step, 1) + 16), "bc_profile_start")
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i % BUFFER_SETS)
    e1.record()
    torch.cuda.synchronize()
    _cabi.lib.bc_profile_stop()
    t_busy_end = time.perf_counter()
    eager_ms = e0.elapsed_time(e1) / args.steps
    import ctypes
    per_kernel = {}
    kid, ms = ctypes.c_int(), ctypes.c_float()
    for i in range(_cabi.lib.bc_profile_count()):
        _cabi.check(_cabi.lib.bc_profile_get(i, ctypes.byref(kid), ctypes.byref(ms)), "bc_profile_get")
        per_kernel.setdefault(_cabi.lib.bc_kernel_name(kid.value).decode(), []).append(ms.value)
    kernels = {k: {"launches": len(v), "mean_us": 1e3 * sum(v) / len(v), "total_ms": sum(v)} for k, v in per_kernel.items()}
    if kernels:
        top = max(kernels, key=lambda k: kernels[k]["total_ms"])
        alg = kernel_algorithmic_bytes(top, N, C, F, h, w)
        peak, peak_src = measured_peak()
        if alg is not None:
            achieved = alg / (kernels[top]["mean_us"] * 1e-6) / 1e9
            traffic = None
            if top in NCU_TRAFFIC:
                b, units = NCU_TRAFFIC[top]
                traffic = b * (N * C * h * w) / units
            roofline = {"bound": "hbm", "kernel": top, "achieved": achieved, "peak": peak, "unit": "GB/s",
                        "frac": achieved / peak, "traffic": traffic, "algorithmic_bytes": alg,
                        "mean_us": kernels[top]["mean_us"], "peak_source": peak_src,
                        "kernels": {k: round(v["mean_us"], 2) for k, v in kernels.items()}}

    # ---- end to end: pinned host buffers in, host results out, through the module
    e2e = None
    stage("end-to-end leg")
    if not args.skip_e2e:
        hx = torch.from_numpy(wl.x).pin_memory()
        hgo = torch.from_numpy(wl.grad_output).pin_memory()
        depth = max(1, args.e2e_depth)
        # batches in flight write to distinct host result buffers
        results = [(torch.empty((N, C * F, h, w), dtype=torch.float32).pin_memory(),
                    torch.empty((N, C, h, w), dtype=torch.float32).pin_memory(),
                    torch.empty((4, C, F), dtype=torch.float32).pin_memory()) for _ in range(depth)]
        hout, hgin, hgp = results[0]
        pipe = bc.HostPipeline(module, N, h, w, chunks=args.e2e_chunks, depth=depth)
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
        if world > 1:
            t = torch.tensor([sec], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            sec = float(t.item())
        e2e = {"value": wl.outputs * world / sec / 1e9, "unit": UNIT,
               "h2d_bytes_per_step": hx.numel() * 4 + hgo.numel() * 4,
               "d2h_bytes_per_step": (hout.numel() + hgin.numel() + hgp.numel()) * 4,
               "ms_per_step": sec * 1e3, "steps": k_e2e, "chunks": args.e2e_chunks, "batches_in_flight": depth,
               "api": "box_convolution.HostPipeline.submit/wait -> bc_boxconv2d_host_step (C ABI, pinned host buffers in and out, "
                      "chunked copy/compute overlap on 3 streams; every batch's inputs go up and its results come back inside the timed region)"}
        t_busy_end = time.perf_counter()

    sampler.stop_flag = True
    sampler.join(timeout=1.0)
    clocks = sampler.summary(t_start, t_end)
    if clocks["samples"] < 3:
        wider = sampler.summary(t_start, t_busy_end)
        wider["window"] = "timed region too short for NVML polling; includes the eager and end-to-end legs"
        clocks = wider

    cpu_baseline = None
    stage("cpu baseline")
    if rank == 0 and world == 1 and not args.skip_cpu_baseline:
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

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": describe(args.workload), "global_batch": N * world, "batch_per_gpu": N,
                       "l2": "rotating %d input/output buffer sets (%.0f MB touched per set)" % (
                           BUFFER_SETS, wl.algorithmic_bytes / 1e6),
                       "launch": "eager" if graphs is None else (
                           "cuda graph replay of clip+forward+backward, %d consecutive steps (one per buffer set) per graph launch" % BUFFER_SETS
                           if multi is not None else
                           "cuda graph replay of clip+forward+backward, one graph per buffer set; all-reduce of step k on a side stream, overlapping step k+1"),
                       "eager_ms_per_step": eager_ms,
                       "collective": "nccl all_reduce of the packed (4,C,F) parameter gradient" if world > 1 else "none"},
            "hbm_gbs_step": wl.algorithmic_bytes * world / (ms_per_step * 1e-3) / 1e9,
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
            "gpu_launches": int(launches_per_step * args.steps), "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    stage("done")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", default="cfg2", choices=sorted(CONFIGS) + ["cfg4", "infer"])
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
