#!/usr/bin/env python
"""Benchmark of the fused dw-conv + BN-inference + quantize path.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl own|reference]
                  [--workload cfg1|cfg0|cfg2|cfg3|cfg4|cfg1q8|ops|bwd|pw1|body] [--batch B] [--scaling weak|strong]

A "step" is one pass of the workload's layer stack over one batch of seeded synthetic
input (cfg1: the 17 depthwise layers of MobileNetV2 at 224x224, batch 256 per GPU, fp32,
each layer followed by BN-inference and FixedPointQuantize(unsigned, n=8, delta=2^-3)).
The batch is sharded by image: with N GPUs every rank runs its own 256 images (weak
scaling), no data-path collective except cfg3's per-channel min/max all-reduce.

One JSON line is printed by rank 0:
  value      whole-job images/s with inputs resident in HBM (CUDA events, max over ranks); the
             17 launches of a step are replayed from a CUDA graph (config.launch)
  e2e        the same through the public call with HOST buffers: pinned-host -> device copy
             of every layer input and device -> host copy of every layer output inside the
             timed region
  roofline   algorithmic bytes of the fused kernels of one step / their measured duration,
             against the measured HBM copy bandwidth (MEASURED_PEAKS.json)
  cpu_baseline  the CPU oracle (a port of the reference's CPU algorithm; nnabla core is not
             installable here) on a bounded sample, all host cores
  other_workloads (N = 1, cfg1 only)  short device-timed passes of cfg0, cfg2, cfg3, cfg4 and the
             five standalone operators, each with its algorithmic GB/s and roofline fraction
--impl reference times that CPU path alone, on the same workload definition.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "nnabla-ext-cuda_b200", "python")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import numpy as np  # noqa: E402

FALLBACK_HBM_GBS = 6650.0


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum, one ncu pass per launch) of the 17
# launches of one cfg1 fp32 step, captured at batch 64 (profiles/cfg1_step_dram_traffic_batch64.md):
# 958.7 MB read (1.001x the algorithmic input bytes) + 171.6 MB written before the kernels
# ended (the remaining output lines are still in the 126 MB L2 then and are written back
# later). The read traffic is proportional to the batch, so the figure is scaled by
# batch / 64; the write share seen before a kernel ends grows with the batch, so the scaled
# figure is a lower bound of the writes (which cannot exceed the output bytes: no re-writes).
CFG1_F32_TRAFFIC_BATCH64 = 958.7e6 + 171.6e6


def measured_traffic(args, batch):
    if args.workload != "cfg1" or args.dtype != "f32" or args.only_layers or args.force_path is not None:
        return None
    return CFG1_F32_TRAFFIC_BATCH64 * batch / 64.0


class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t_begin=None, t_end=None):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        inside = [ln for (t, ln) in self.lines if t_begin is None or (t_begin <= t <= t_end + 0.05)]
        if len(inside) < 2:  # a very short region: fall back to everything sampled around it
            inside = [ln for (_, ln) in self.lines]
        for ln in inside:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def host_threads():
    """Cores this process may run on (torchrun sets OMP_NUM_THREADS=1, which the oracle's
    explicit thread count overrides)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def make_cpu_pass(specs, sample_n, nthreads):
    """Returns a function that runs the unfused CPU chain (dw-conv, BN, quantizer: three
    passes, like the reference's CPU functions) of the whole layer stack once on
    `sample_n` seeded images and returns the seconds it took."""
    from dwbnq import workloads
    from oracle import oracle
    datas = []
    for s in specs:
        small = workloads.LayerSpec(s.name, sample_n, s.c, s.h, s.w, s.k, s.stride, s.pad, s.quant, s.seed, s.x_dist)
        datas.append((small, workloads.make_layer_data(small)))

    def one_pass():
        t0 = time.perf_counter()
        for small, d in datas:
            q = workloads.quant_for_ops(small, d)
            oracle.fused_layer(d["x"], d["w"], d["b"], d["beta"], d["gamma"], d["mean"], d["var"], small.bn_eps,
                               (small.stride,) * 2, (small.pad,) * 2, q, nthreads=nthreads)
        return time.perf_counter() - t0

    return one_pass


def cpu_stack_images_per_s(specs, sample_n, nthreads, min_seconds):
    """Repeats the CPU pass until `min_seconds` are spent; (images/s, seconds per pass, passes)."""
    one_pass = make_cpu_pass(specs, sample_n, nthreads)
    one_pass()  # untimed: page in the buffers, start the thread pool
    total, passes = 0.0, 0
    while passes == 0 or (total < min_seconds and passes < 1000):
        total += one_pass()
        passes += 1
    return sample_n * passes / total, total / passes, passes


def run_reference(args):
    """The reference arm: the reference's CPU algorithm (oracle port) on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from dwbnq import workloads
    from oracle import oracle
    oracle.build()
    specs = workloads.workload(args.workload, args.batch)
    nthreads = host_threads()
    sample_n = args.cpu_sample
    one_pass = make_cpu_pass(specs, sample_n, nthreads)
    times = []
    for i in range(args.warmup + args.steps):
        dt = one_pass()
        if i >= args.warmup:
            times.append(dt)
    total = sum(times)
    value = sample_n * len(times) / total
    bytes_per_image = sum(s.algorithmic_bytes(4, 1) for s in specs)
    line = {
        "impl": "reference", "metric": "images_per_s", "value": value, "unit": "images/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args), "sample": "%d images per step" % sample_n},
        "cpu_baseline": {"value": value, "unit": "images/s", "cores": nthreads, "kind": "port",
                         "sample": "%d images of the layer stack per step, unfused 3-function chain" % sample_n,
                         "effective_gbs": value * bytes_per_image / 1e9},
        "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_name(args):
    names = {"cfg0": "cfg0 single layer [B,64,56,56] 3x3 s1 + BN + FixedPointQuantize(sign,n=8,2^-4)",
             "cfg1": "cfg1 MobileNetV2 17 depthwise 3x3 layers @224 + BN + FixedPointQuantize(unsigned,n=8,2^-3)",
             "cfg2": "cfg2 [B,144,56,56] 5x5 s1 + BN + Pow2Quantize(sign,with_zero,n=8,m=1)",
             "cfg3": "cfg3 [B,192,28,28] 3x3 s2 + BN + MinMaxQuantize(per-channel, batch-inclusive)",
             "cfg4": "cfg4 = cfg1 in fp16",
             "cfg1q8": "cfg1 with 8-bit storage: inputs are uint8 codes of FixedPointQuantize(unsigned,n=8,2^-5) of the "
                       "cfg1 activations, outputs the uint8 codes of the layer's FixedPointQuantize(unsigned,n=8,2^-3)"}
    return names[args.workload]


def standalone_op_rows(torch, ops, device, n, half, warmup, reps):
    """Times the five standalone operators on one [n, 96, 56, 56] activation, L2 flushed
    before every timed launch. Rows of {layer, ms, gbs, bytes}; the algorithmic bytes are
    2 * itemsize per element (read once, write once), and 3 * itemsize for MinMaxQuantize (a
    read for the per-channel min / max, then a read and a write for the quantize step)."""
    tdtype = torch.float16 if half else torch.float32
    itemsize = 2 if half else 4
    c, hw = 96, 56
    g = torch.Generator(device="cpu").manual_seed(0)
    x = torch.randn((n, c, hw, hw), generator=g, dtype=torch.float32).to(device).to(tdtype)
    w = (torch.randn((c, 3, 3), generator=g) / 3).to(device).to(tdtype)
    vec = lambda lo, hi: (torch.rand(c, generator=g) * (hi - lo) + lo).to(device).to(tdtype)
    b, mean, var, gamma, beta = vec(-.3, .3), vec(-.3, .3), vec(.5, 1.5), vec(.8, 1.2), vec(-.3, .3)
    y = torch.empty_like(x)
    qr_min, qr_max = torch.zeros(c, device=device, dtype=tdtype), torch.ones(c, device=device, dtype=tdtype)
    ql_min, ql_max = torch.zeros(c, device=device, dtype=tdtype), torch.full((c,), 255.0, device=device, dtype=tdtype)
    ws = ops.workspace(c, device)
    calls = [
        ("DepthwiseConvolution 3x3 s1", lambda: ops.depthwise_convolution(x, w, b, 1, (1, 1), (1, 1), out=y)),
        ("BatchNormalization(batch_stat=False)", lambda: ops.batch_normalization(x, beta, gamma, mean, var, out=y)),
        ("FixedPointQuantize(sign,n=8,2^-4)", lambda: ops.fixed_point_quantize(x, True, 8, 2.0 ** -4, out=y)),
        ("Pow2Quantize(sign,with_zero,n=8,m=1)", lambda: ops.pow2_quantize(x, True, True, 8, 1, out=y)),
        ("MinMaxQuantize(per-channel, x_min_max)", lambda: ops.min_max_quantize(
            x, qr_min, qr_max, ql_min, ql_max, x_min_max=True, ws=ws, out=y)),
    ]
    rows = []
    for name, fn in calls:
        for _ in range(warmup):
            fn()
        ts = []
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(reps):
            flush_l2(torch, device)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ms = float(np.median(ts))
        nbytes = (3 if name.startswith("MinMax") else 2) * x.numel() * itemsize
        rows.append({"layer": name, "ms": ms, "gbs": nbytes / ms / 1e6, "elements": x.numel(), "bytes": nbytes})
    ops.check_device_flag()
    return rows


def backward_op_rows(torch, ops, device, n, warmup, reps):
    """The training-side kernels on [n, 96, 56, 56] fp32, L2 flushed before every timed launch:
    the straight-through backward of the two quantizers (x and dy read, dx written: 3 * 4 bytes
    per element) and the convolution's gradients (input gradient: dy read, dx written; weight
    and bias gradients: x and dy read)."""
    c, hw = 96, 56
    g = torch.Generator(device="cpu").manual_seed(1)
    x = torch.randn((n, c, hw, hw), generator=g).to(device)
    dy = torch.randn((n, c, hw, hw), generator=g).to(device)
    w = (torch.randn((c, 3, 3), generator=g) / 3).to(device)
    dx, dw, db = torch.empty_like(x), torch.empty_like(w), torch.empty(c, device=device)
    e = x.numel() * 4
    calls = [
        ("FixedPointQuantize backward (fine-grained STE)", 3 * e,
         lambda: ops.fixed_point_quantize_backward(dy, x, True, 8, 2.0 ** -4, True, dx=dx)),
        ("Pow2Quantize backward (fine-grained STE)", 3 * e,
         lambda: ops.pow2_quantize_backward(dy, x, True, True, 8, 1, True, dx=dx)),
        ("DepthwiseConvolution 3x3 s1 backward: input gradient", 2 * e,
         lambda: ops.depthwise_convolution_backward(x, w, dy, 1, (1, 1), (1, 1), dx=dx, need=(True, False, False))),
        ("DepthwiseConvolution 3x3 s1 backward: weight and bias gradients", 2 * e,
         lambda: ops.depthwise_convolution_backward(x, w, dy, 1, (1, 1), (1, 1), dw=dw, db=db, need=(False, True, True))),
    ]
    rows = []
    for name, nbytes, fn in calls:
        for _ in range(warmup):
            fn()
        ts = []
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(reps):
            flush_l2(torch, device)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ms = float(np.median(ts))
        rows.append({"layer": name, "ms": ms, "gbs": nbytes / ms / 1e6, "bytes": nbytes})
    ops.check_device_flag()
    return rows


def run_standalone_ops(args):
    """The five standalone operators on one [B, 96, 56, 56] activation (308 MB at the default
    B = 256, fp32): per-operator time and algorithmic GB/s (2 * B bytes per element: read
    once, write once). One JSON line in the bench format; `layers` holds the operators."""
    import torch
    from dwbnq import ops
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the dwbnq path has no CPU fallback")
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    half = args.dtype == "f16"
    itemsize = 2 if half else 4
    n, c, hw = args.batch, 96, 56
    peak, peak_kind = measured_peak()
    if args.workload == "bwd":  # the training-side kernels on the same activation (fp32)
        rows = backward_op_rows(torch, ops, device, n, args.warmup, max(3, min(args.steps, 20)))
    else:
        rows = standalone_op_rows(torch, ops, device, n, half, args.warmup, max(3, min(args.steps, 20)))
    total_ms = sum(r["ms"] for r in rows)
    bytes_all = sum(r["bytes"] for r in rows)
    achieved = bytes_all / total_ms / 1e6
    line = {"metric": "images_per_s", "value": n / (total_ms / 1e3), "unit": "images/s", "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
            "config": {"workload": ("bwd: the backward kernels on [%d,%d,%d,%d]" if args.workload == "bwd" else
                                    "ops: the five standalone operators on [%d,%d,%d,%d]") % (n, c, hw, hw),
                       "l2": "L2 flushed before every timed launch"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "peak_kind": peak_kind}, "gpu_launches": None, "layers": rows}
    print(json.dumps(line), flush=True)


def run_pointwise(args):
    """Workload pw1 alone: the 33 pointwise layers around cfg1's depthwise layers at batch B
    (default 256), one JSON line in the bench format; `layers` holds the per-layer rows and the
    two summary rows. --only-layers restricts the pass (profiling)."""
    import torch
    from dwbnq import ops, workloads
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the dwbnq path has no CPU fallback")
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    peak, peak_kind = measured_peak()
    n = args.batch or 256
    if args.only_layers:
        keep = {int(i) for i in args.only_layers.split(",")}
        full = workloads.pw1
        workloads.pw1 = lambda b=256: [sp for i, sp in enumerate(full(b)) if i in keep]
    rows = pointwise_rows(torch, ops, workloads, device, n, peak)
    tot = [r for r in rows if r["workload"].startswith("pw1: ") and r["workload"].endswith("fp32")][0]
    line = {"metric": "images_per_s", "value": tot["images_per_s"], "unit": "images/s", "n_gpus": 1, "steps": 10,
            "warmup": 2, "ms_per_step": tot["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": "pw1: the pointwise convolutions of MobileNetV2 around the depthwise layers, batch %d, "
                                   "each fused with BN, activation and FixedPointQuantize" % n,
                       "l2": "L2 flushed before every timed launch"},
            "roofline": {"bound": "hbm", "achieved": tot["gbs"], "peak": peak, "unit": "GB/s", "frac": tot["frac"],
                         "traffic": None, "peak_kind": peak_kind}, "gpu_launches": sum(1 for r in rows if r["workload"].startswith("pw1.l")), "layers": rows}
    print(json.dumps(line), flush=True)


def body_row(torch, ops, workloads, device, batch, peak, reps=10, half=False):
    """The 50 layers of MobileNetV2's body as ONE network: the unfused function list nnabla would
    build (166 functions), fused by the two graph passes into 17 FusedDwBnQuant + 33
    FusedPwBnQuant nodes, every layer reading the previous layer's output; pointwise parameters
    prepared once, the 50 launches replayed from a CUDA graph, L2 flushed before each replay."""
    from dwbnq import graph
    nodes, host, x_in, x_out, _ = workloads.body_graph(batch)
    shapes = {k: v.shape for k, v in host.items()}
    fused = graph.fuse_pw_bn_quant(graph.fuse_dw_bn_quant(nodes, [x_out], shapes), [x_out], shapes)
    tensors = {k: torch.from_numpy(v).to(device) for k, v in host.items()}
    if half:  # binary16 tensors (the 8-bit activations are exact in binary16; the parameters are rounded to it)
        tensors = {k: v.half() for k, v in tensors.items()}
    del host
    runner = graph.GraphRunner(fused, tensors)
    runner.replay()
    runner.synchronize()
    ts = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(reps):
        flush_l2(torch, device)
        e0.record()
        runner.replay()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    runner.synchronize()
    ms = float(np.median(ts))
    nbytes = sum(sp.algorithmic_bytes(2 if half else 4, batch) for _, sp in workloads.mobilenetv2_body(batch))
    flops = sum(sp.flops(batch) for kind, sp in workloads.mobilenetv2_body(batch) if kind == "pw")
    out_shape = tuple(tensors[x_out].shape)
    del runner, tensors
    torch.cuda.empty_cache()
    return {"workload": "body: MobileNetV2's 50 depthwise + pointwise layers chained (each reads the previous output), "
                        "fused by the graph passes" + (", binary16 tensors" if half else ""),
            "dtype": "f16" if half else "f32", "batch": batch, "ms": ms, "best_ms": float(min(ts)),
            "images_per_s": batch / (ms / 1e3), "gbs": nbytes / ms / 1e6, "frac": nbytes / ms / 1e6 / peak,
            "tflops": flops / ms / 1e9, "algorithmic_bytes": nbytes, "launches": len(fused), "output": list(out_shape),
            "kernel": "fused_plane_* (17 launches) + pw_tc_kernel (33 launches)",
            "timing": "median of %d CUDA-graph replays of the 50 launches, L2 flushed before each" % reps}


def run_body(args):
    """Workload body alone: one JSON line in the bench format."""
    import torch
    from dwbnq import ops, workloads
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the dwbnq path has no CPU fallback")
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    peak, peak_kind = measured_peak()
    row = body_row(torch, ops, workloads, device, args.batch, peak, half=args.dtype == "f16")
    line = {"metric": "images_per_s", "value": row["images_per_s"], "unit": "images/s", "n_gpus": 1, "steps": 10,
            "warmup": 3, "ms_per_step": row["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": row["dtype"], "data": "synthetic", "config": {"workload": row["workload"], "batch": args.batch,
                                                            "l2": "L2 flushed before every timed replay"},
            "roofline": {"bound": "hbm", "achieved": row["gbs"], "peak": peak, "unit": "GB/s", "frac": row["frac"],
                         "traffic": None, "peak_kind": peak_kind}, "gpu_launches": row["launches"], "layers": [row]}
    print(json.dumps(line), flush=True)


def bind_to_gpu_numa_node(torch, index):
    """Restricts this process to the CPUs of the NUMA node its GPU hangs off, so that the
    pinned host buffers of the end-to-end pass (allocated afterwards, first touched here) are
    local to the GPU's PCIe root. Returns the node, or None when the topology is not exposed."""
    try:
        p = torch.cuda.get_device_properties(index)
        bdf = "%04x:%02x:%02x.0" % (p.pci_domain_id, p.pci_bus_id, p.pci_device_id)
        with open("/sys/bus/pci/devices/%s/numa_node" % bdf) as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open("/sys/devices/system/node/node%d/cpulist" % node) as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if len(allowed) >= 2:
            os.sched_setaffinity(0, allowed)
            return node
    except Exception:
        pass
    return None


FAMILY = {0: "fused_generic_kernel", 1: "fused_tiled_kernel (cooperative fill)", 2: "fused_tiled_kernel (TMA)",
          3: "fused_tiled_kernel (bulk copy)", 4: "fused_plane_* kernels", 5: "fused_plane_gen_kernel"}


def pointwise_rows(torch, ops, workloads, device, batch, peak):
    """The 33 pointwise convolutions around cfg1's depthwise layers (workload pw1), each fused with
    BN, its activation and its FixedPointQuantize, one layer at a time with its own seeded input
    resident in HBM; the layer's parameters are prepared once (dwbnq_pwconv_prepare) and a timed
    step is the one kernel of dwbnq_pwconv_fused_fwd_prepared. Every launch is replayed from a CUDA graph with L2 flushed before it (the
    deeper layers move less than L2 holds); median of 10. Per-layer rows for the fp32-accurate
    three-pass TF32 mode, and a summary row for it and for the single-pass TF32 mode."""
    rows, totals = [], {"fp32": [0.0, 0, 0.0], "tf32": [0.0, 0, 0.0]}
    lib_ms = {"conv": 0.0, "chain": 0.0}
    half_ms = 0.0
    import torch.nn.functional as F
    tf32_was = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False

    def median_ms(fn, reps=5, graph=False):
        fn()
        if graph:
            g = torch.cuda.CUDAGraph()
            cap = torch.cuda.Stream(device)
            cap.wait_stream(torch.cuda.current_stream(device))
            with torch.cuda.stream(cap):
                fn()
                with torch.cuda.graph(g, stream=cap):
                    fn()
            torch.cuda.current_stream(device).wait_stream(cap)
            fn = g.replay
            fn()
        ts = []
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(reps):
            flush_l2(torch, device)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return float(np.median(ts))

    for spec in workloads.pw1(batch):
        d = workloads.make_pointwise_data(spec)
        t = {k: torch.from_numpy(v).to(device) for k, v in d.items()}
        del d
        y = torch.empty((batch, spec.c_out, spec.h, spec.h), dtype=torch.float32, device=device)
        ws = ops.pwconv_workspace(t["x"], t["w"])
        path = ops.pwconv_plan(t["x"], t["w"])
        for math in ("fp32", "tf32"):
            if math == "tf32" and path == 0:
                ms = rows[-1]["ms"]  # the FMA kernel has one mode
            else:
                # inference: the parameters are prepared once (dwbnq_pwconv_prepare), a step is one launch
                ops.pwconv_prepare(t["x"], t["w"], t["b"], t["beta"], t["gamma"], t["mean"], t["var"], spec.bn_eps,
                                   act=spec.act, math=math, ws=ws)

                def call():
                    ops.fused_pw_bn_quant_prepared(t["x"], t["w"], ws, True, spec.quant, spec.act, math=math, out=y)
                call()
                g = torch.cuda.CUDAGraph()
                cap = torch.cuda.Stream(device)
                cap.wait_stream(torch.cuda.current_stream(device))
                with torch.cuda.stream(cap):
                    call()
                    with torch.cuda.graph(g, stream=cap):
                        call()
                torch.cuda.current_stream(device).wait_stream(cap)
                g.replay()
                torch.cuda.synchronize()
                ts = []
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                for _ in range(10):
                    flush_l2(torch, device)
                    e0.record()
                    g.replay()
                    e1.record()
                    torch.cuda.synchronize()
                    ts.append(e0.elapsed_time(e1))
                ms = float(np.median(ts))
                del g
            nbytes = spec.algorithmic_bytes(4, batch)
            totals[math][0] += ms
            totals[math][1] += nbytes
            totals[math][2] += spec.flops(batch)
            if math == "fp32":
                rows.append({"workload": "%s %d->%d @%dx%d" % (spec.name, spec.c_in, spec.c_out, spec.h, spec.h), "dtype": "f32",
                             "batch": batch, "ms": ms, "images_per_s": batch / (ms / 1e3), "gbs": nbytes / ms / 1e6,
                             "frac": nbytes / ms / 1e6 / peak, "tflops": spec.flops(batch) / ms / 1e9,
                             "algorithmic_bytes": nbytes,
                             "kernel": "pw_tc_kernel (tcgen05, three TF32 passes)" if path == 1 else "pw_simt_kernel (FMA)",
                             "timing": "median of 10 CUDA-graph replays, L2 flushed before each"})
        # the same layer on binary16 tensors (binary16 MMAs behind TMA where rows are 16-byte multiples, else one exact
        # TF32 pass on gathered rows): per-layer time beside the fp32 row, and a summary row
        th = {k: v.half() for k, v in t.items()}
        yh = torch.empty((batch, spec.c_out, spec.h, spec.h), dtype=torch.float16, device=device)
        ops.pwconv_prepare(th["x"], th["w"], th["b"], th["beta"], th["gamma"], th["mean"], th["var"], spec.bn_eps,
                           act=spec.act, ws=ws)
        ms16 = median_ms(lambda: ops.fused_pw_bn_quant_prepared(th["x"], th["w"], ws, True, spec.quant, spec.act, out=yh),
                         reps=7, graph=True)
        half_ms += ms16
        rows[-1]["ms_f16"] = ms16
        del th, yh
        # library baseline: the convolution as cuDNN runs it in fp32 (TF32 off, as the reference
        # defaults), then BN, activation and quantizer as the separate passes the reference makes
        lib_ms["conv"] += median_ms(lambda: F.conv2d(t["x"], t["w"], t["b"]))
        q = spec.quant

        def chain():
            v = F.conv2d(t["x"], t["w"], t["b"])
            ops.batch_normalization(v, t["beta"], t["gamma"], t["mean"], t["var"], eps=spec.bn_eps, out=v)
            if spec.act == "relu6":
                v.clamp_(0.0, 6.0)
            ops.fixed_point_quantize(v, q["sign"], q["n"], q["delta"], out=v)
        lib_ms["chain"] += median_ms(chain)
        del t, y, ws
        torch.cuda.empty_cache()
    torch.backends.cudnn.allow_tf32 = tf32_was
    ops.check_device_flag()
    nb_all, fl_all = totals["fp32"][1], totals["fp32"][2]
    for key, what in (("conv", "torch conv2d alone (cuDNN fp32, TF32 off)"),
                      ("chain", "torch conv2d (cuDNN fp32) + BN + ReLU6 + FixedPointQuantize as separate passes")):
        ms = lib_ms[key]
        rows.append({"workload": "pw1 library baseline: " + what, "dtype": "f32", "batch": batch, "ms": ms,
                     "images_per_s": batch / (ms / 1e3), "gbs": nb_all / ms / 1e6, "frac": nb_all / ms / 1e6 / peak,
                     "tflops": fl_all / ms / 1e9, "algorithmic_bytes": nb_all, "kernel": "library kernels, for comparison only",
                     "timing": "median of 5 eager calls per layer, L2 flushed before each (host launch overhead included)"})
    rows.append({"workload": "pw1: 33 pointwise layers, fp16 tensors", "dtype": "f16", "batch": batch, "ms": half_ms,
                 "images_per_s": batch / (half_ms / 1e3), "gbs": nb_all / 2 / half_ms / 1e6, "frac": nb_all / 2 / half_ms / 1e6 / peak,
                 "tflops": fl_all / half_ms / 1e9, "algorithmic_bytes": nb_all // 2, "kernel": "pw_tc_kernel<half> (kind::f16 behind TMA on 16-byte rows, else gathered with one exact TF32 pass)",
                 "timing": "median of 7 CUDA-graph replays per layer, L2 flushed before each"})
    for math, (ms, nbytes, fl) in totals.items():
        rows.append({"workload": "pw1: 33 pointwise layers, math %s" % math, "dtype": "f32", "batch": batch, "ms": ms,
                     "images_per_s": batch / (ms / 1e3), "gbs": nbytes / ms / 1e6, "frac": nbytes / ms / 1e6 / peak,
                     "tflops": fl / ms / 1e9, "algorithmic_bytes": nbytes, "kernel": "sum of the per-layer medians",
                     "timing": "median of 10 CUDA-graph replays per layer, L2 flushed before each"})
    return rows


def other_workloads(torch, ops, workloads, device, cfg1_layers, args):
    """Short device-timed passes of the configurations that are not the headline workload
    (cfg0, cfg2, cfg3, cfg4) and of the five standalone operators, each with its algorithmic
    bytes against the measured copy bandwidth. Inputs are resident in HBM; cfg0's 51 MB
    working set would stay in L2, so L2 is flushed before each of its timed launches; the
    others move more than L2 holds per step and are replayed from a CUDA graph."""
    peak, _ = measured_peak()
    out = []

    def timed(name, dtype_name, batch, specs, tensors, flush, extra=None):
        tdtype = torch.float16 if dtype_name == "f16" else torch.float32
        itemsize = 2 if dtype_name == "f16" else 4
        lay = []
        for s, t in zip(specs, tensors):
            y = torch.empty((batch, s.c, s.ho, s.wo), dtype=tdtype, device=device)
            q = workloads.quant_for_ops(s, t)
            ws = ops.workspace(s.c, device) if s.quant["kind"] == "minmax" else None
            lay.append((s, t, y, q, ws))

        def step():
            for s, t, y, q, ws in lay:
                ops.fused_dw_bn_quant(t["x"], t["w"], t["b"], t["beta"], t["gamma"], t["mean"], t["var"], s.bn_eps,
                                      pad=(s.pad, s.pad), stride=(s.stride, s.stride), quant=q, ws=ws, out=y)

        for _ in range(3):
            step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if flush:
            ts = []
            for _ in range(10):
                flush_l2(torch, device)
                e0.record()
                step()
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1))
            ms, how = float(np.median(ts)), "median of 10 launches, L2 flushed before each"
        else:
            g = torch.cuda.CUDAGraph()
            cap = torch.cuda.Stream(device)
            cap.wait_stream(torch.cuda.current_stream(device))
            with torch.cuda.stream(cap):
                step()
                with torch.cuda.graph(g, stream=cap):
                    step()
            torch.cuda.current_stream(device).wait_stream(cap)
            for _ in range(3):
                g.replay()
            torch.cuda.synchronize()
            reps = 50
            e0.record()
            for _ in range(reps):
                g.replay()
            e1.record()
            torch.cuda.synchronize()
            ms, how = e0.elapsed_time(e1) / reps, "mean of %d CUDA-graph replays" % reps
        ops.check_device_flag()
        nbytes = sum(s.algorithmic_bytes(itemsize, batch) for s in specs)
        s0 = specs[0]
        plan = ops.fused_plan(tensors[0]["x"], tensors[0]["w"], lay[0][2], pad=(s0.pad, s0.pad),
                              stride=(s0.stride, s0.stride))
        row = {"workload": name, "dtype": dtype_name, "batch": batch, "ms": ms, "images_per_s": batch / (ms / 1e3),
               "gbs": nbytes / ms / 1e6, "frac": nbytes / ms / 1e6 / peak, "algorithmic_bytes": nbytes,
               "kernel": FAMILY.get(plan["path"], "?") if len(specs) == 1 else "fused_plane_* kernels (17 launches)",
               "timing": how}
        if extra:
            row.update(extra)
        out.append(row)

    def on_device(spec, n, tdtype):
        d = workloads.make_layer_data(spec, n=n)
        return {k: torch.from_numpy(v).to(device).to(tdtype) for k, v in d.items()}

    s = workloads.cfg0()
    timed("cfg0", "f32", 32, s, [on_device(s[0], 32, torch.float32)], flush=True)
    s = workloads.cfg2()
    timed("cfg2", "f32", 128, s, [on_device(s[0], 128, torch.float32)], flush=False)
    s = workloads.cfg3()
    timed("cfg3", "f32", 512, s, [on_device(s[0], 512, torch.float32)], flush=False,
          extra={"note": "one GPU, no collective; two passes (reduce + store fp32, quantize in place): "
                         "executed bytes 4*(E_in + 3*E_out), gbs counts the compulsory 4*(E_in + E_out)"})
    if args.dtype == "f32" and cfg1_layers and cfg1_layers[0][0].n == 256:
        # cfg4 = the cfg1 tensors cast to fp16
        specs = [l[0] for l in cfg1_layers]
        tens = [{k: v.half() for k, v in l[2].items()} for l in cfg1_layers]
        timed("cfg4", "f16", 256, specs, tens, flush=False)
        del tens
        # cfg1q8 = cfg1 with one-byte activations in and out (FixedPointQuantize codes), fp32 parameters
        in_delta = 2.0 ** -5
        lay8 = []
        for sp, _, t, *_ in cfg1_layers:
            xq = torch.clamp(torch.floor(t["x"] / in_delta + 0.5), 0, 255).to(torch.uint8)
            y8 = torch.empty((256, sp.c, sp.ho, sp.wo), dtype=torch.uint8, device=device)
            lay8.append((sp, t, xq, y8, workloads.quant_for_ops(sp, t)))

        def step8():
            for sp, t, xq, y8, q in lay8:
                ops.fused_dw_bn_quant_code8(xq, in_delta, t["w"], t["b"], t["beta"], t["gamma"], t["mean"], t["var"], sp.bn_eps,
                                            pad=(sp.pad, sp.pad), stride=(sp.stride, sp.stride), quant=q, out=y8)
        for _ in range(3):
            step8()
        g8 = torch.cuda.CUDAGraph()
        cap = torch.cuda.Stream(device)
        cap.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(cap):
            step8()
            with torch.cuda.graph(g8, stream=cap):
                step8()
        torch.cuda.current_stream(device).wait_stream(cap)
        for _ in range(3):
            g8.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(50):
            g8.replay()
        e1.record()
        torch.cuda.synchronize()
        ops.check_device_flag()
        ms8 = e0.elapsed_time(e1) / 50
        nb8 = sum(sp.algorithmic_bytes(1, 256) for sp in specs)
        out.append({"workload": "cfg1q8", "dtype": "f32 arithmetic, u8 storage", "batch": 256, "ms": ms8,
                    "images_per_s": 256 / (ms8 / 1e3), "gbs": nb8 / ms8 / 1e6, "frac": nb8 / ms8 / 1e6 / peak,
                    "algorithmic_bytes": nb8, "kernel": "fused_plane_* kernels, 8-bit storage (17 launches)",
                    "timing": "mean of 50 CUDA-graph replays",
                    "note": "a quarter of cfg1's bytes: bound by the fp32 arithmetic, not by HBM"})
        del lay8, g8
    for r in standalone_op_rows(torch, ops, device, 256, False, 3, 10):
        out.append({"workload": "op: " + r["layer"], "dtype": "f32", "batch": 256, "ms": r["ms"],
                    "images_per_s": 256 / (r["ms"] / 1e3), "gbs": r["gbs"], "frac": r["gbs"] / peak,
                    "algorithmic_bytes": r["bytes"], "kernel": "standalone operator on [256,96,56,56]",
                    "timing": "median of 10 launches, L2 flushed before each"})
    for r in backward_op_rows(torch, ops, device, 256, 3, 10):
        out.append({"workload": "bwd: " + r["layer"], "dtype": "f32", "batch": 256, "ms": r["ms"],
                    "images_per_s": 256 / (r["ms"] / 1e3), "gbs": r["gbs"], "frac": r["gbs"] / peak,
                    "algorithmic_bytes": r["bytes"], "kernel": "training-side kernel on [256,96,56,56]",
                    "timing": "median of 10 launches, L2 flushed before each"})
    torch.cuda.empty_cache()
    out.extend(pointwise_rows(torch, ops, workloads, device, 256, peak))
    out.append(body_row(torch, ops, workloads, device, 256, peak))
    out.append(body_row(torch, ops, workloads, device, 256, peak, half=True))
    torch.cuda.empty_cache()
    return out


def run_own(args):
    import torch
    import torch.distributed as dist
    from dwbnq import ops, workloads
    from dwbnq.comm import Communicator

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the dwbnq path has no CPU fallback")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    numa = bind_to_gpu_numa_node(torch, local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    half = args.workload == "cfg4" or args.dtype == "f16"
    code8 = args.workload == "cfg1q8"  # activations travel as one-byte codes, parameters stay fp32
    tdtype = torch.float16 if half else torch.float32
    itemsize = 1 if code8 else (2 if half else 4)
    in_delta = 2.0 ** -5
    # weak scaling (default): --batch images on every GPU. strong: --batch is the GLOBAL batch,
    # split evenly, so the total work stays fixed as GPUs are added.
    if args.scaling == "strong":
        if args.batch % world:
            raise SystemExit("--scaling strong needs a global batch divisible by the GPU count")
        batch = args.batch // world
    else:
        batch = args.batch
    specs = workloads.workload(args.workload, batch)
    if args.only_layers:
        specs = [specs[int(i)] for i in args.only_layers.split(",")]
    need_comm = any(s.quant["kind"] == "minmax" for s in specs) and world > 1
    comm = Communicator.from_torch_distributed(device) if need_comm else None

    # ---- seeded inputs: this rank's images of the global batch, in pinned host memory ----
    layers = []
    for s in specs:
        d = workloads.make_layer_data(s, n=batch, first_image=rank * batch)
        pin = (lambda t: t) if args.no_e2e else (lambda t: t.pin_memory())  # pinned only when it is copied from
        host = {k: pin(torch.from_numpy(v).to(tdtype)) for k, v in d.items()}
        if code8:  # the layer input as the previous layer would have left it: FixedPointQuantize codes
            xq = np.clip(np.floor(d["x"] / np.float32(in_delta) + np.float32(0.5)), 0, 255).astype(np.uint8)
            host["x"] = pin(torch.from_numpy(xq))
        devt = {k: v.to(device, non_blocking=True) for k, v in host.items()}
        ydt = torch.uint8 if code8 else tdtype
        y = torch.empty((batch, s.c, s.ho, s.wo), dtype=ydt, device=device)
        y_host = None if args.no_e2e else torch.empty(y.shape, dtype=ydt).pin_memory()
        if args.no_e2e:
            host = {"x": host["x"][:0]}  # the device copies are all that is needed
        q = workloads.quant_for_ops(s, devt)
        ws = ops.workspace(s.c, device) if s.quant["kind"] == "minmax" else None
        layers.append((s, host, devt, y, y_host, q, ws))
    torch.cuda.synchronize()

    def launch(layer, x=None, use_comm=True):
        s, _, t, y, _, q, ws = layer
        if args.ablate:  # profiling only: drop BN and / or the quantizer to attribute instruction counts
            bn = None if "bn" in args.ablate else t
            qq = None if "quant" in args.ablate else q
            ops.fused_dw_bn_quant(t["x"], t["w"], t["b"], bn and bn["beta"], bn and bn["gamma"], bn and bn["mean"],
                                  bn and bn["var"], s.bn_eps, pad=(s.pad, s.pad), stride=(s.stride, s.stride),
                                  quant=qq, out=y)
            return
        if code8:
            ops.fused_dw_bn_quant_code8(t["x"], in_delta, t["w"], t["b"], t["beta"], t["gamma"], t["mean"], t["var"],
                                        s.bn_eps, pad=(s.pad, s.pad), stride=(s.stride, s.stride), quant=q, out=y)
            return
        ops.fused_dw_bn_quant(t["x"] if x is None else x, t["w"], t["b"], t["beta"], t["gamma"], t["mean"], t["var"],
                              s.bn_eps, pad=(s.pad, s.pad), stride=(s.stride, s.stride), quant=q,
                              comm=comm if use_comm else None, ws=ws, out=y)

    def step_eager():
        for layer in layers:
            launch(layer)

    # The launches of one step are captured once into a CUDA graph and replayed (--no-graph:
    # launched one by one from the host). The library's entry points only set attributes and
    # launch, so they can be captured once their first-call set-up has run in the warm-up.
    graph = None

    def step():
        if graph is not None:
            graph.replay()
        else:
            step_eager()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    launches_per_step = sum(2 if s.quant["kind"] == "minmax" else 1 for s in specs)

    if args.tune:
        ops.set_tuning(*[int(v) for v in args.tune.split(",")])
    if args.force_path is not None:
        ops.set_forced_path(args.force_path)

    # ---- device-resident timing ---------------------------------------------------------
    for _ in range(args.warmup):
        step()
    barrier()
    if args.graph and comm is None:
        cap = torch.cuda.Stream(device)
        cap.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(cap):
            step_eager()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=cap):
                step_eager()
        torch.cuda.current_stream(device).wait_stream(cap)
        graph = g
        for _ in range(3):
            step()
        barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    # events every `chunk` steps inside the one timed region: the value is total / steps (mean);
    # the chunks give the median and the best step beside it
    chunk = 5 if args.steps >= 10 else 1
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps // chunk + 2)]
    t_begin = time.time()
    marks[0].record()
    n_marks = 1
    for i in range(args.steps):
        step()
        if (i + 1) % chunk == 0 or i + 1 == args.steps:
            marks[n_marks].record()
            n_marks += 1
    barrier()
    t_end = time.time()
    elapsed_ms = marks[0].elapsed_time(marks[n_marks - 1])
    chunk_ms = [marks[j].elapsed_time(marks[j + 1]) / chunk for j in range(args.steps // chunk)]
    # A short timed region sees too few of the 50 ms clock samples: keep the same load running,
    # untimed, until 0.4 s of it have been sampled.
    while comm is None and time.time() - t_begin < 0.4:  # (steps with a collective must stay in lock step)
        step()
        torch.cuda.synchronize()
        t_end = time.time()
    barrier()
    clocks = sampler.stop(t_begin, t_end) if rank == 0 else None
    ops.check_device_flag()

    # ---- MinMax with a collective: where the step's time goes ------------------------------
    # (a) the two passes alone (every rank reduces and quantizes with its own shard's ranges),
    # (b) the bare all-reduce(max) of the 2*C packed floats, back to back on the stream; the
    # step itself, timed above, is (a) + pack kernel + all-reduce in between.
    phase_ms = [0.0, 0.0]
    if comm is not None:
        def loop_ms(fn, reps=50):
            for _ in range(3):
                fn()
            barrier()
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            for _ in range(reps):
                fn()
            a1.record()
            barrier()
            return a0.elapsed_time(a1) / reps

        phase_ms[0] = loop_ms(lambda: [launch(layer, use_comm=False) for layer in layers])
        buf = torch.zeros(2 * max(s.c for s in specs), device=device, dtype=torch.float32)
        phase_ms[1] = loop_ms(lambda: comm.allreduce_max_(buf))

    # ---- per-layer durations (separate pass, same launches; for the roofline breakdown) ----
    per_layer = []
    for layer in ([] if args.no_layer_pass else layers):
        s = layer[0]
        reps = max(3, min(args.steps, 10))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ts = []
        for _ in range(reps):
            flush_l2(torch, device)
            e0.record()
            launch(layer)
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ms = float(np.median(ts))
        per_layer.append({"layer": s.name, "c": s.c, "hw": s.h, "stride": s.stride, "ms": ms,
                          "gbs": s.algorithmic_bytes(itemsize, batch) / ms / 1e6})

    # ---- end to end: host buffers in, host buffers out ------------------------------------
    # Every layer's input comes from pinned host memory and every layer's result goes back to
    # pinned host memory inside the timed region. Uploads, kernels and downloads run on three
    # streams chained by events (PCIe is full duplex), the way a caller with host tensors
    # would drive the library.
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    compute = torch.cuda.current_stream(device)
    up, down = torch.cuda.Stream(device), torch.cuda.Stream(device)
    ev_in = [torch.cuda.Event() for _ in layers]
    ev_done = [torch.cuda.Event() for _ in layers]
    ev_out = [torch.cuda.Event() for _ in layers]
    first = [True]

    def e2e_step(kernels=True):
        for i, layer in enumerate(layers):
            s, host, t, y, y_host, q, ws = layer
            with torch.cuda.stream(up):
                if not first[0]:
                    up.wait_event(ev_done[i])  # last step's kernel has consumed the old input
                t["x"].copy_(host["x"], non_blocking=True)
                ev_in[i].record(up)
            compute.wait_event(ev_in[i])
            if not first[0]:
                compute.wait_event(ev_out[i])  # last step's result has left the output buffer
            if kernels:
                launch(layer)
            ev_done[i].record(compute)
            with torch.cuda.stream(down):
                down.wait_event(ev_done[i])
                y_host.copy_(y, non_blocking=True)
                ev_out[i].record(down)
        first[0] = False

    def e2e_join():
        compute.wait_stream(up)
        compute.wait_stream(down)

    if not args.no_e2e:
        e2e_step()
        e2e_join()
    barrier()
    t0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(0 if args.no_e2e else e2e_steps):
        e2e_step()
    e2e_join()
    e1.record()
    barrier()
    e2e_ms = max(e0.elapsed_time(e1), 0.0)
    e2e_wall_ms = 1e3 * (time.perf_counter() - t0)
    # The same copies on the same three streams with the same event chain and NO kernel: how
    # fast the box moves these bytes at this N. e2e close to it = bound by the copies.
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c0.record()
    for _ in range(0 if args.no_e2e else e2e_steps):
        e2e_step(kernels=False)
    e2e_join()
    c1.record()
    barrier()
    copy_ms = max(c0.elapsed_time(c1), 0.0)
    h2d = sum(l[1]["x"].numel() * itemsize for l in layers)
    d2h = sum(l[3].numel() * itemsize for l in layers)

    # ---- the other configurations and the standalone operators (N = 1, cfg1 runs only) --------
    other = None
    if world == 1 and args.workload == "cfg1" and not args.no_other and not args.only_layers and \
            args.force_path is None and not args.ablate:
        other = other_workloads(torch, ops, workloads, device, layers, args)

    # ---- max over ranks ---------------------------------------------------------------------
    if world > 1:
        tt = torch.tensor([elapsed_ms, e2e_ms, copy_ms] + phase_ms + chunk_ms, device=device, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        elapsed_ms, e2e_ms, copy_ms = float(tt[0]), float(tt[1]), float(tt[2])
        phase_ms = [float(tt[3]), float(tt[4])]
        chunk_ms = [float(v) for v in tt[5:]]

    if rank == 0:
        images = batch * world * args.steps
        value = images / (elapsed_ms / 1e3)
        bytes_per_step = sum(s.algorithmic_bytes(itemsize, batch) for s in specs)
        peak, peak_kind = measured_peak()
        ms_per_step = elapsed_ms / args.steps
        achieved = bytes_per_step / (ms_per_step / 1e3) / 1e9
        from oracle import oracle
        oracle.build()
        nthreads = host_threads()
        # the CPU baseline is timed at N = 1 only (at N > 1 the other ranks would sit idle for it)
        skip_cpu = args.no_cpu or world > 1
        cpu_ips, cpu_dt, cpu_passes = (None, 0.0, 0) if skip_cpu else cpu_stack_images_per_s(
            specs, args.cpu_sample, nthreads, args.cpu_seconds)
        # the same chain on one core (nnabla's CPU functions are plain loops), 8 images
        cpu_1core = None if skip_cpu else cpu_stack_images_per_s(specs, 8, 1, 2.0)[0]
        bytes_per_image = sum(s.algorithmic_bytes(4, 1) for s in specs)
        line = {
            "metric": "images_per_s", "value": value, "unit": "images/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step,
            "ms_per_step_median": float(np.median(chunk_ms)) if chunk_ms else ms_per_step,
            "ms_per_step_best": float(min(chunk_ms)) if chunk_ms else ms_per_step,
            "higher_is_better": True, "scaling": args.scaling,
            "vs_baseline": None, "dtype": "f16" if half else "f32", "data": "synthetic",
            "storage": "uint8 codes" if code8 else ("f16" if half else "f32"),
            "config": {"workload": workload_name(args), "batch_per_gpu": batch, "global_batch": batch * world,
                       "layers": len(specs), "parallelism": "batch-sharded x%d" % world, "numa_node": numa, "launch": "cuda graph" if graph is not None else "stream",
                       "l2": "per-step working set %.1f GB >> 126 MB L2; every layer has its own buffers"
                             % (bytes_per_step / 1e9)},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": measured_traffic(args, batch), "peak_kind": peak_kind,
                         "frac_of_nominal_8000": achieved / 8000.0,
                         "kernel": "fused_plane_kernel + fused_plane_s2_kernel (all %d launches of a step, per GPU)"
                                   % launches_per_step,
                         "algorithmic_bytes_per_step": bytes_per_step},
            "cpu_baseline": {"value": cpu_ips, "unit": "images/s", "cores": nthreads, "kind": "port",
                             "sample": ("not timed: measured at N = 1 only" if world > 1 else
                                        "%d images of the layer stack, unfused 3-function chain, %d passes of %.2f s"
                                        % (args.cpu_sample, cpu_passes, cpu_dt)),
                             "effective_gbs": None if cpu_ips is None else cpu_ips * bytes_per_image / 1e9,
                             "value_one_core": cpu_1core},
            "e2e": {"value": None if args.no_e2e else batch * world * e2e_steps / (e2e_ms / 1e3), "unit": "images/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "wall_ms_per_step": e2e_wall_ms / e2e_steps,
                    "copy_only": None if args.no_e2e else {
                        "value": batch * world * e2e_steps / (copy_ms / 1e3), "unit": "images/s",
                        "gbs_per_gpu": (h2d + d2h) * e2e_steps / (copy_ms / 1e3) / 1e9,
                        "what": "the same host<->device copies, streams and events without the kernels"}},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
            "layers": per_layer,
        }
        if other is not None:
            line["other_workloads"] = other
        if comm is not None:
            line["phases"] = {"step_ms": ms_per_step, "two_passes_without_collective_ms": phase_ms[0],
                              "allreduce_max_alone_ms": phase_ms[1],
                              "collective_share_of_step": max(0.0, 1.0 - phase_ms[0] / ms_per_step),
                              "what": "max over ranks; the collective is one ncclAllReduce(max) of 2*C floats "
                                      "between the reduce pass and the quantize pass"}
        print(json.dumps(line), flush=True)
    if comm is not None:
        comm.destroy()
    if world > 1:
        dist.destroy_process_group()


_flush_buf = {}


def flush_l2(torch, device):
    """Overwrites a 512 MB buffer (4x the 126 MB L2) so the next launch starts cold."""
    b = _flush_buf.get(device)
    if b is None:
        b = torch.empty(512 * 1024 * 1024, dtype=torch.uint8, device=device)
        _flush_buf[device] = b
    b.fill_(1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
    ap.add_argument("--workload", default="cfg1", choices=["cfg0", "cfg1", "cfg2", "cfg3", "cfg4", "cfg1q8", "ops", "bwd", "pw1", "body"])
    ap.add_argument("--batch", type=int, default=None, help="images per GPU (default: the workload's batch)")
    ap.add_argument("--dtype", default="f32", choices=["f32", "f16"])
    ap.add_argument("--cpu-sample", type=int, default=None, help="images per CPU-baseline pass")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="CPU time spent on the cpu_baseline sample")
    ap.add_argument("--e2e-steps", type=int, default=3)
    # reduced runs for profiling a single kernel (the printed line is then not a bench result)
    ap.add_argument("--only-layers", default="", help="comma-separated layer indices of the workload")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-layer-pass", action="store_true")
    ap.add_argument("--no-other", action="store_true", help="skip the short passes of the other configurations")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="weak: --batch images per GPU; strong: --batch is the global batch, split over the GPUs")
    ap.add_argument("--ablate", default="", help="profiling only: 'bn', 'quant' or 'bn,quant' are left out")
    ap.add_argument("--no-graph", dest="graph", action="store_false",
                    help="launch every kernel from the host instead of replaying the step from a CUDA graph")
    ap.add_argument("--force-path", type=int, default=None, help="profiling only: kernel family 0..4")
    ap.add_argument("--tune", default="", help="profiling only: planner override P,row_blocks,threads,rows_per_patch")
    args = ap.parse_args()
    defaults = {"cfg0": 32, "cfg1": 256, "cfg2": 128, "cfg3": 512, "cfg4": 256, "cfg1q8": 256, "ops": 256, "bwd": 256, "pw1": 256, "body": 256}
    if args.batch is None:
        args.batch = defaults[args.workload]
    if args.warmup < 3:
        args.warmup = 3
    if args.cpu_sample is None:
        args.cpu_sample = {"cfg0": 32, "cfg1": 64, "cfg2": 32, "cfg3": 128, "cfg4": 64, "cfg1q8": 64,
                           "ops": 0, "bwd": 0, "pw1": 0, "body": 0}[args.workload]
    if args.workload in ("ops", "bwd"):
        run_standalone_ops(args)
    elif args.workload == "pw1":
        run_pointwise(args)
    elif args.workload == "body":
        run_body(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_own(args)


if __name__ == "__main__":
    main()
