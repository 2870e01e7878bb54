#!/usr/bin/env python
"""Benchmark of the int8 conv / fc hot path: whole-network inference throughput.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--net resnet50|mobilenet_v1]
                    [--batch-per-gpu B] [--impl ours|reference]

One "step" is one forward pass of the int8 network over a batch of B images on each GPU
(weak scaling: the batch is sharded by image, weights are replicated, no collective on the
data path).  Prints ONE JSON line on rank 0:

  value      images/s over all GPUs, inputs resident in HBM, timed with CUDA events on the
             launching stream (max over ranks)
  e2e        the same with host buffers: every step copies that step's fp32 images from pinned
             host memory and reads the logits back (copies overlap the previous step's compute)
  roofline   of the dominant kernel (the tcgen05 implicit GEMM): algorithmic bytes of its
             launches in a step (every conv/fc layer after the stem) / their measured duration,
             against the measured HBM peak (and against the nominal 8 TB/s), plus the tensor-core
             view of the same launches and of the compute-bound class (the 3x3 convolutions)
  cpu_baseline  the reference's own x86 int8 path (oracle/_ref, built from the reference
             sources) on a bounded sample of the same workload, all host threads
  extra      the other benchmark configurations, measured in the same process: MobileNetV1 at 32 and
             256 images per GPU, ResNet-50 at global batch 1024 on one GPU, the per-layer table (single
             3x3 layer, fc sweep, depthwise, sparse_conv sweep), a sustained figure (graph replays for
             about two seconds) and the step without CUDA graphs (`--no-extras` skips all of these)

`--impl reference` times only that CPU path and prints the same line shape.
"""
import argparse
import importlib
import json
import os
import statistics
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "paddle-lite_b200"))

DEFAULT_BATCH = {"resnet50": 128, "mobilenet_v1": 32}


INT8_PEAK_TOPS = 4500.0   # dense int8 datasheet figure
HBM_NOMINAL_GBS = 8000.0  # "about 8 TB/s" of the benchmark definition


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def bind_to_gpu_numa_node(nvml_index):
    """Runs this process on the CPUs NVML reports as local to the GPU, so that the pinned host buffers
    allocated afterwards come from the memory next to the GPU's PCIe root.  Reads topology only; sets
    nothing on the GPU.  Returns the number of CPUs bound to, or None when NVML cannot tell."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(nvml_index)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        cpus = {64 * i + b for i, wd in enumerate(mask) for b in range(64) if (wd >> b) & 1}
        allowed = os.sched_getaffinity(0)
        cpus &= allowed
        if cpus and cpus != allowed:
            os.sched_setaffinity(0, cpus)
        return len(cpus) if cpus else None
    except Exception:
        return None


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU while a timed region runs (NVML reads
    from a background thread every few milliseconds; nothing is ever set)."""

    def __init__(self, index):
        self.index, self.samples, self.stop_flag, self.thread, self.err = index, [], False, None, None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception as exc:  # no NVML: report that instead of inventing numbers
            self.err = str(exc)
            return
        self.thread = threading.Thread(target=self._poll, daemon=True)
        self.thread.start()
        # the first NVML reads of a process are slow (library and driver set-up): let them happen before anything is timed
        t0 = time.perf_counter()
        while len(self.samples) < 3 and self.err is None and time.perf_counter() - t0 < 1.0:
            time.sleep(0.005)

    def _poll(self):
        nv = self.nv
        while not self.stop_flag:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)
                reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle) \
                    if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons") \
                    else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                self.samples.append((time.perf_counter(), mhz, reasons))
            except Exception as exc:
                self.err = str(exc)
                return
            time.sleep(0.004)

    def stop(self, t_begin=None, t_end=None):
        self.stop_flag = True
        if self.thread:
            self.thread.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["clock sampling unavailable: %s" % self.err],
                    "samples": 0}
        sel = [s for s in self.samples if (t_begin is None or s[0] >= t_begin) and (t_end is None or s[0] <= t_end)]
        if not sel:  # region shorter than one poll: take the sample closest to it
            mid = 0.5 * ((t_begin or 0) + (t_end or 0))
            sel = [min(self.samples, key=lambda s: abs(s[0] - mid))]
        nv = self.nv
        names = {"hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4)}
        seen = set()
        for _, _, bits in sel:
            for name, mask in names.items():
                if bits & mask:
                    seen.add(name)
        return {"sm_mhz": statistics.median([s[1] for s in sel]), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(seen), "samples": len(sel)}


def _nvml_index(local_rank):
    """NVML enumerates physical GPUs; honour CUDA_VISIBLE_DEVICES when it lists ordinals."""
    vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
    ids = [v.strip() for v in vis.split(",") if v.strip()]
    if local_rank < len(ids) and ids[local_rank].isdigit():
        return int(ids[local_rank])
    return local_rank


def layer_bytes(spec, batch):
    """Algorithmic bytes of the conv/fc launches of one step (int8 or fp32 tensors read and
    written once, weights once) and their multiply-accumulates."""
    c, h, w = spec["image"]
    hw = {"x": (h, w)}
    total_bytes, macs, launches = 0, 0, 0
    per_layer = []
    # projection shortcuts that run inside the block's last launch
    shortcuts = importlib.import_module("paddle-lite_b200.networks").fusable_shortcuts(spec)
    if os.environ.get("PLB_FUSE_BLOCKS", "1") == "0":
        shortcuts = {}
    for op in spec["ops"]:
        if op["op"] == "conv" and op["dst"] in shortcuts:
            ih, iw = hw[op["src"]]
            hw[op["dst"]] = ((ih - 1) // op["s"] + 1, (iw - 1) // op["s"] + 1)
            continue
        if op["op"] in ("conv", "conv_add_relu"):
            ih, iw = hw[op["src"]]
            oh, ow = (ih + 2 * op["p"] - op["k"]) // op["s"] + 1, (iw + 2 * op["p"] - op["k"]) // op["s"] + 1
            groups = op.get("groups", 1)
            b = batch * ih * iw * op["cin"] + op["cout"] * (op["cin"] // groups) * op["k"] ** 2 + 8 * op["cout"]
            if op["op"] == "conv":
                b += batch * oh * ow * op["cout"] * (1 if op["out"] == "i8" else 4)
                hw[op["dst"]] = (oh, ow)
            else:
                if op["residual"] in shortcuts:
                    # fused block tail: the shortcut's input pixels and filter instead of a residual tensor
                    sc = shortcuts[op["residual"]]
                    b += batch * oh * ow * sc["cin"] + sc["cout"] * sc["cin"] + 8 * sc["cout"]
                else:
                    b += batch * oh * ow * op["cout"] * 4  # residual read
                for key, size in (("dst_f32", 4), ("dst_i8", 1)):
                    if op[key]:
                        b += batch * oh * ow * op["cout"] * size
                        hw[op[key]] = (oh, ow)
            m = batch * oh * ow * op["cout"] * (op["cin"] // groups) * op["k"] ** 2
            if op["op"] == "conv_add_relu" and op["residual"] in shortcuts:
                m += batch * oh * ow * op["cout"] * shortcuts[op["residual"]]["cin"]
            if groups == 1 and op["src"] != "x":  # the stem runs with its staging kernel in the head
                total_bytes += b
                macs += m
                launches += 1
            per_layer.append((op["name"], b, m, groups))
        elif op["op"] == "maxpool":
            ih, iw = hw[op["src"]]
            hw[op["dst"]] = ((ih + 2 * op["p"] - op["k"]) // op["s"] + 1, (iw + 2 * op["p"] - op["k"]) // op["s"] + 1)
        elif op["op"] == "fc":
            total_bytes += batch * op["k"] + op["k"] * op["n"] + batch * op["n"] * 4 + 8 * op["n"]
            macs += batch * op["k"] * op["n"]
            launches += 1
    return total_bytes, macs, launches, per_layer


# --------------------------------------------------------------------------- CPU reference arm
def cpu_reference_prepare(qnet, threads):
    """PrepareForRun of every conv layer on the reference objects (filter packing, scale folding), one kernel
    instance per host thread: done once, outside the timed region, as the reference does."""
    from oracle import oracle as O
    spec, layers, scales = qnet["spec"], qnet["layers"], qnet["scales"]
    c, h, w = spec["image"]
    hw = {"x": (h, w)}
    prepared = {}
    for op in spec["ops"]:
        if op["op"] in ("conv", "conv_add_relu"):
            L = layers[op["name"]]
            out_s = float(scales[op["dst"]]) if op["op"] == "conv" and op["out"] == "i8" else None
            rc = O.RefConv(L["wq"], L["ws"], float(scales[op["src"]]), L["bias"], op.get("act", 0), 0.0, out_scale=out_s,
                           in_hw=hw[op["src"]], stride=(op["s"],) * 2, pads=(op["p"],) * 4, groups=op.get("groups", 1),
                           threads=threads)
            prepared[op["name"]] = rc
            for key in ("dst", "dst_f32", "dst_i8"):
                if op.get(key):
                    hw[op[key]] = (rc.ho, rc.wo)
        elif op["op"] == "maxpool":
            ih, iw = hw[op["src"]]
            hw[op["dst"]] = ((ih + 2 * op["p"] - op["k"]) // op["s"] + 1, (iw + 2 * op["p"] - op["k"]) // op["s"] + 1)
    return prepared


def cpu_reference_pass(qnet, images, threads, prepared):
    """One forward pass through the reference's own x86 objects (im2col + gemm_s8u8, built from
    the reference sources into oracle/_ref), conv and fc layers; fp32 glue in numpy/torch."""
    import torch
    import torch.nn.functional as F
    from oracle import oracle as O
    spec, layers, scales = qnet["spec"], qnet["layers"], qnet["scales"]
    t = {"x": O.calib_f32_to_i8(images, float(scales["x"]))}
    for op in spec["ops"]:
        kind = op["op"]
        if kind == "conv":
            t[op["dst"]] = prepared[op["name"]].run(t[op["src"]])
        elif kind == "conv_add_relu":
            y = prepared[op["name"]].run(t[op["src"]])
            s = np.maximum(y + t[op["residual"]], np.float32(0))
            if op["dst_f32"]:
                t[op["dst_f32"]] = s
            if op["dst_i8"]:
                t[op["dst_i8"]] = O.calib_f32_to_i8(s, float(scales[op["dst_i8"]]))
        elif kind == "maxpool":
            x = torch.from_numpy(t[op["src"]].astype(np.float32))
            t[op["dst"]] = F.max_pool2d(x, op["k"], op["s"], op["p"]).numpy().astype(np.int8)
        elif kind == "avgpool_calib":
            avg = t[op["src"]].mean(axis=(2, 3), dtype=np.float32)
            t[op["dst"]] = O.calib_f32_to_i8(avg, float(scales[op["dst"]]))
        elif kind == "fc":
            L = layers[op["name"]]
            t[op["dst"]] = O.ref_fc_int8(t[op["src"]], L["wq"], L["ws"], float(scales[op["src"]]), L["bias"])
    return t["logits"]


def cpu_baseline(qnet, spec, sample_images, repeats=1, prepared=None):
    from oracle import oracle as O
    threads = os.cpu_count() or 1
    kind = "reference" if O.ref_available() else "port"
    rng = np.random.default_rng(5)
    images = rng.standard_normal((sample_images,) + spec["image"]).astype(np.float32)
    if kind == "port":  # exact-integer restatement when the reference objects are absent
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import net_oracle
        fn = lambda: net_oracle.forward(qnet, images)  # noqa: E731
    else:
        if prepared is None:
            prepared = cpu_reference_prepare(qnet, threads)
        fn = lambda: cpu_reference_pass(qnet, images, threads, prepared)  # noqa: E731
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        fn()
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return {"value": sample_images / best, "unit": "images/s", "cores": threads, "kind": kind,
            "sample": "%d images, whole %s forward (all conv/fc layers through the x86 int8 path, layers prepared "
                      "once outside the timed region, batch sharded over %d host threads), best of %d"
                      % (sample_images, spec["name"], threads, repeats),
            "seconds": best}


# --------------------------------------------------------------------------- main
def graph_of(torch, stream, fn):
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        fn()
    return g


def time_replays(torch, stream, graph, steps, sync):
    """ms per replay, CUDA events on the launching stream."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    e0.record(stream)
    for _ in range(steps):
        graph.replay()
    e1.record(stream)
    sync()
    return e0.elapsed_time(e1) / steps


def tc_launches(runner, only_3x3=False):
    """Enqueues the tensor-core launches of a step after the stem (same buffers, same order)."""
    for st in runner.steps[1:]:
        if st[0] == "conv" and st[1].desc.groups == 1:
            if only_3x3 and st[1].desc.kh != 3:
                continue
            st[1].run_nhwc(runner.buf[st[2]], out=runner.buf[st[3]])
        elif only_3x3:
            continue
        elif st[0] == "conv_add_relu":
            _, conv, src, res, df, dq, next_s = st
            conv.run_nhwc_add_relu(runner.buf[src], runner.buf[res], next_s, want_f32=df is not None,
                                   out_f32=runner.buf[df] if df else None, out_i8=runner.buf[dq] if dq else None)
        elif st[0] == "block_add_relu":
            _, conv, src, sc_conv, sc_src, df, dq, next_s = st
            conv.run_nhwc_block_add_relu(runner.buf[src], sc_conv, runner.buf[sc_src], next_s,
                                         want_f32=df is not None, out_f32=runner.buf[df] if df else None,
                                         out_i8=runner.buf[dq] if dq else None)
        elif st[0] == "dwpw":
            st[1].run_nhwc_dwpw(st[2], runner.buf[st[3]], out=runner.buf[st[4]])
        elif st[0] == "fc":
            st[1].run(runner.buf[st[2]], out=runner.buf[st[3]])


def measure_network(torch, plb, networks, ctx, stream, net, batch, steps, warmup, micro_batch=None):
    """Device-resident images/s of one network at one batch on this GPU (graph replays)."""
    spec = networks.SPECS[net]()
    qnet = networks.build_quantized(spec, seed=1234, calib_images=16, device="cuda")
    runner = networks.Runner(plb, ctx, qnet, batch, micro_batch=micro_batch)
    images = torch.randn(runner.image_shape, device="cuda")
    with torch.cuda.stream(stream):
        n0 = ctx.launch_count()
        runner.forward(images)
        ctx.sync()
        launches = ctx.launch_count() - n0
        g = graph_of(torch, stream, lambda: runner.forward(images))
        for _ in range(warmup):
            g.replay()
        ms = time_replays(torch, stream, g, steps, torch.cuda.synchronize)
        # the same step without a CUDA graph: what a caller of Run() per layer gets
        for _ in range(2):
            runner.forward(images)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(max(steps // 2, 3)):
            runner.forward(images)
        e1.record(stream)
        torch.cuda.synchronize()
        eager_ms = e0.elapsed_time(e1) / max(steps // 2, 3)
        ctx.sync()
    out = {"workload": "%s, batch %d%s" % (spec["name"], batch, (" in slices of %d" % micro_batch) if micro_batch else ""),
           "value": batch / (ms / 1e3), "unit": "images/s", "ms_per_step": ms, "eager_ms_per_step": eager_ms,
           "launches_per_step": int(launches), "steps": steps}
    del runner, images, g
    torch.cuda.empty_cache()
    return out


def layer_table(plb, ctx):
    """The per-layer configurations of the benchmark: single 3x3 layer, fc sweep, depthwise, sparse_conv sweep."""
    import layer_bench as LB
    L = LB.Layers(plb, ctx, iters=20, warm=0.1)
    vendor = L.int8_peak(4096)
    vt = vendor["TOPS"]
    rows = [vendor, L.int8_peak(8192)]
    rows.append(L.conv(64, 56, 64, 3, 1, 1, 1, "f32", nchw=True))        # the single-layer config, NCHW in / fp32 out
    rows.append(L.conv(64, 56, 64, 3, 1, 1, 128, "i8"))                  # the same layer at the network's batch
    for cin, hw in ((128, 28), (256, 14), (512, 7)):
        rows.append(L.conv(cin, hw, cin, 3, 1, 1, 128, "i8"))
    for cin, hw in ((64, 56), (128, 28), (256, 14), (512, 7)):
        rows.append(L.conv(cin, hw, cin, 3, 1, 1, 1024, "i8"))           # the same layers in launches of 1024 images
    for m, k, n in LB.FC_SWEEP:
        for out in ("f32", "i8"):
            rows.append(L.fc(m, k, n, out, int8_measured_tops=vt))
    for cin, hw, stride in ((32, 112, 1), (64, 112, 2), (128, 56, 1), (512, 14, 1)):
        rows.append(L.conv(cin, hw, cin, 3, stride, 1, 256, "i8", groups=cin))
    for cin, cout, hw, stride in ((32, 64, 112, 1), (64, 128, 112, 2), (128, 128, 56, 1), (256, 256, 28, 1)):
        rows.append(L.dwpw(cin, cout, hw, stride, 256))                  # MobileNetV1 blocks: depthwise + 1x1 in one launch
    for cin, cout, hw in LB.SPARSE_SWEEP:
        rows.append(L.sparse(cin, cout, hw, 256, False, False, "auto"))
        rows.append(L.sparse(cin, cout, hw, 256, False, True, "auto"))
    rows.append(L.sparse(32, 64, 112, 256, True, False, "walk"))
    rows.append(L.sparse(128, 128, 56, 256, True, False, "walk"))
    for r in rows:
        r.pop("hbm_peak", None)
        if "tensor_frac_of_vendor_gemm" not in r and r["ops"] and "cublaslt" not in r["layer"]:
            r["tensor_frac_of_vendor_gemm"] = round(r["TOPS"] / vt, 3)
    return rows, vt


# DRAM read + write bytes as a fraction of the algorithmic bytes, per class of tensor-core launch, from single-launch
# ncu captures of one layer of each class at the benchmark's batch (dram__bytes_read.sum + dram__bytes_write.sum of
# `layer_bench.py` commands).  Traffic below the algorithmic bytes means that a tensor written by one launch is still in
# the 126 MB L2 when it ends; none of the classes re-reads.  bench.py scales each layer's algorithmic bytes by its
# class's ratio to estimate the DRAM traffic of a step; only ResNet-50 at 128 images per GPU has captures behind it.
TRAFFIC_RATIO = {"residual": 899.3 / 950.6,    # conv + fp32 residual + ReLU + calib, 64 -> 256 @ 56 x 56
                 "block_tail": 508.3 / 565.2,  # the same with the shortcut GEMM inside
                 "pointwise": 108.6 / 128.5,   # 1x1, int8 out, 256 -> 64 @ 56 x 56
                 "conv3x3": 25.9 / 51.4}       # 3x3, int8 out, 64 -> 64 @ 56 x 56 (window mode)


def estimated_traffic(spec, batch, per_layer, shortcuts):
    """DRAM bytes per tensor-core launch of a step, estimated per class (see TRAFFIC_RATIO); None without captures."""
    if spec["name"] != "resnet50_v1.5" or batch != 128:
        return None
    ops = {op["name"]: op for op in spec["ops"] if "name" in op}
    total, n = 0.0, 0
    for name, b, m, groups in per_layer:
        op = ops[name]
        if groups != 1 or op.get("src") == "x":
            continue
        if op["op"] == "conv_add_relu":
            cls = "block_tail" if op["residual"] in shortcuts else "residual"
        else:
            cls = "conv3x3" if op["k"] == 3 else "pointwise"
        total += b * TRAFFIC_RATIO[cls]
        n += 1
    return (total / n, total) if n else None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=0, help="timed steps (0 = 100; 20 for --impl reference)")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--net", default="resnet50", choices=sorted(DEFAULT_BATCH))
    ap.add_argument("--batch-per-gpu", type=int, default=0)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-sample", type=int, default=0, help="images in the CPU baseline sample (0 = auto)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="only the headline workload")
    args = ap.parse_args()
    if args.steps <= 0:
        # long enough that the one image copy nothing overlaps (the first of the timed region) is 1 % of the run
        args.steps = 20 if args.impl == "reference" else 100
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    per_gpu = args.batch_per_gpu or DEFAULT_BATCH[args.net]
    warmup = max(args.warmup, 3)

    networks = importlib.import_module("paddle-lite_b200.networks")
    sharding = importlib.import_module("paddle-lite_b200.sharding")
    # weak scaling: the global batch grows with the number of GPUs; rank r owns a contiguous slice of it
    global_batch = per_gpu * args.gpus
    lo, hi = sharding.shard_slice(global_batch, rank if world > 1 else 0, max(world, 1))
    batch = hi - lo if world > 1 else per_gpu
    spec = networks.SPECS[args.net]()
    workload = "%s int8 PTQ, 224x224, batch %d per GPU" % (spec["name"], per_gpu)
    base = {"metric": "int8 %s inference throughput" % spec["name"], "unit": "images/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": warmup, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int8 x int8 -> int32 (fp32 epilogue)",
            "data": "synthetic: seeded N(0,1) fp32 images, He-init weights quantised per channel, "
                    "activation scales from a 16-image calibration pass",
            "config": {"workload": workload, "global_batch": global_batch, "parallelism":
                       "batch-sharded replicas (dp%d), no collective" % args.gpus,
                       "l2": "per-step activations (>1 GB) exceed the 126 MB L2; no explicit flush"}}

    if args.impl == "reference":
        if rank != 0:
            return
        import torch
        torch.set_num_threads(os.cpu_count() or 1)
        qnet = networks.build_quantized(spec, seed=1234, calib_images=4, device="cpu")
        # one step = 4 images per host thread (≈ 2-3 s of CPU work), so the default 3 + 20 steps take about a minute
        sample = args.cpu_sample or 4 * max(os.cpu_count() or 1, 8)
        times = []
        from oracle import oracle as O
        prepared = cpu_reference_prepare(qnet, os.cpu_count() or 1) if O.ref_available() else None
        for i in range(warmup + args.steps):
            cb = cpu_baseline(qnet, spec, sample, prepared=prepared)
            if i >= warmup:
                times.append(cb["seconds"])
            if sum(times) > 240:
                break
        ms = 1e3 * sum(times) / len(times)
        val = sample / (ms / 1e3)
        cb.update(value=val)
        cb.pop("seconds", None)
        line = dict(base, impl="reference", value=val, ms_per_step=ms, steps=len(times),
                    cpu_baseline=cb, e2e={"value": val, "unit": "images/s", "h2d_bytes_per_step": 0,
                                           "d2h_bytes_per_step": 0},
                    gpu_launches=0)
        line["config"] = dict(base["config"], workload=workload + " (CPU sample: %d images per step)" % sample)
        print(json.dumps(line))
        return

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference "
                         "for the CPU arm")
    numa_cpus = bind_to_gpu_numa_node(_nvml_index(local_rank))  # before any pinned allocation
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    sys.path.insert(0, os.path.join(ROOT, "paddle-lite_b200"))
    import build as plb_build
    if rank == 0:
        plb_build.build()
    if world > 1:
        dist.barrier()
    plb = importlib.import_module("paddle-lite_b200")

    stream = torch.cuda.Stream()
    copy_stream = torch.cuda.Stream()
    ctx = plb.Context(local_rank, stream=stream)
    qnet = networks.build_quantized(spec, seed=1234, calib_images=16, device="cuda")
    runner = networks.Runner(plb, ctx, qnet, batch)
    rng = np.random.default_rng(1000 + rank)
    host_images = torch.from_numpy(rng.standard_normal(runner.image_shape).astype(np.float32)).pin_memory()
    host_logits = [torch.empty((batch, 1000), dtype=torch.float32).pin_memory() for _ in range(2)]
    dev_images = [host_images.cuda(), torch.empty(runner.image_shape, device="cuda")]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.cuda.stream(stream):
        n0 = ctx.launch_count()
        runner.forward(dev_images[0])       # eager pass: sets kernel attributes, checks for faults
        ctx.sync()
        launches_per_step = ctx.launch_count() - n0
        g_full = graph_of(torch, stream, lambda: runner.forward(dev_images[0]))
        g_body = graph_of(torch, stream, runner.forward_body)
        g_tc = graph_of(torch, stream, lambda: tc_launches(runner))       # the dominant kernel's launches alone
        has_3x3 = any(st[0] == "conv" and st[1].desc.groups == 1 and st[1].desc.kh == 3 for st in runner.steps[1:])
        g_3x3 = graph_of(torch, stream, lambda: tc_launches(runner, only_3x3=True)) if has_3x3 else None

        # ---- device-resident throughput
        sampler = ClockSampler(_nvml_index(local_rank))
        sampler.start()
        for _ in range(5):  # settle a fresh process (first replays of a new graph, clocks) before the warm-up proper
            g_full.replay()
        torch.cuda.synchronize()
        for _ in range(warmup):
            g_full.replay()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t_begin = time.perf_counter()
        e0.record(stream)
        for _ in range(args.steps):
            g_full.replay()
        e1.record(stream)
        barrier()
        t_end = time.perf_counter()
        clocks = sampler.stop(t_begin, t_end)
        value, ms_total = sharding.aggregate_throughput(batch * args.steps, e0.elapsed_time(e1))
        ms_step = ms_total / args.steps

        # ---- dominant kernel alone, and the compute-bound class (3x3 convolutions) alone
        for _ in range(2):
            g_tc.replay()
        tc_ms_step = time_replays(torch, stream, g_tc, args.steps, torch.cuda.synchronize)
        c3_ms_step = None
        if g_3x3 is not None:
            for _ in range(2):
                g_3x3.replay()
            c3_ms_step = time_replays(torch, stream, g_3x3, args.steps, torch.cuda.synchronize)

        # ---- end to end: pinned host images in, logits out, every step.  Two device image buffers: the
        # copy of step i+1 runs while step i computes.
        ev_h2d = [torch.cuda.Event() for _ in range(2)]
        ev_head = [torch.cuda.Event() for _ in range(2)]
        ev_body, ev_d2h = torch.cuda.Event(), torch.cuda.Event()
        d2h_stream = torch.cuda.Stream()

        def e2e_steps(n):
            for i in range(n):
                b = i & 1
                with torch.cuda.stream(copy_stream):
                    if i >= 2:
                        copy_stream.wait_event(ev_head[b])  # this image buffer has been consumed (two steps ago)
                    dev_images[b].copy_(host_images, non_blocking=True)
                    ev_h2d[b].record(copy_stream)
                stream.wait_event(ev_h2d[b])
                runner.forward_head(dev_images[b])
                ev_head[b].record(stream)
                if i >= 1:
                    stream.wait_event(ev_d2h)  # the logits of the step before have left the buffer
                g_body.replay()
                # the result leaves on its own stream: the next step's first layer does not queue behind the copy
                ev_body.record(stream)
                with torch.cuda.stream(d2h_stream):
                    d2h_stream.wait_event(ev_body)
                    host_logits[b].copy_(runner.buf["logits"], non_blocking=True)
                    ev_d2h.record(d2h_stream)
            if n:
                stream.wait_event(ev_d2h)  # the timed region ends when the last result is in host memory

        e2e_steps(warmup)
        barrier()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record(stream)
        e2e_steps(args.steps)
        s1.record(stream)
        barrier()
        e2e_value, e2e_ms_total = sharding.aggregate_throughput(batch * args.steps, s0.elapsed_time(s1))
        e2e_ms_step = e2e_ms_total / args.steps

        # ---- the copies alone (all ranks at once, no kernels): the ceiling of the end-to-end number
        barrier()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record(copy_stream)
        with torch.cuda.stream(copy_stream):
            for i in range(args.steps):
                dev_images[i & 1].copy_(host_images, non_blocking=True)
        c1.record(copy_stream)
        barrier()
        _, h2d_ms_total = sharding.aggregate_throughput(batch * args.steps, c0.elapsed_time(c1))
        h2d_ms = h2d_ms_total / args.steps
        ctx.sync()

    total_bytes, macs, n_tc, per_layer = layer_bytes(spec, batch)
    peak, peak_kind = measured_peaks()
    achieved = total_bytes / (tc_ms_step / 1e3) / 1e9
    fused = networks.fusable_shortcuts(spec) if os.environ.get("PLB_FUSE_BLOCKS", "1") != "0" else {}
    traffic = estimated_traffic(spec, batch, per_layer, fused)
    tensor_tops = 2.0 * macs / (tc_ms_step / 1e3) / 1e12
    h2d_bytes = host_images.numel() * 4
    line = dict(base, value=value, ms_per_step=ms_step, clocks=clocks,
                e2e={"value": e2e_value, "unit": "images/s", "h2d_bytes_per_step": h2d_bytes,
                     "d2h_bytes_per_step": batch * 1000 * 4, "ms_per_step": e2e_ms_step,
                     "h2d_only_ms": h2d_ms, "h2d_gbs_per_rank": h2d_bytes / (h2d_ms / 1e3) / 1e9,
                     "ceiling_images_per_s": args.gpus * batch / (max(h2d_ms, ms_step) / 1e3),
                     "host_cpus_bound": numa_cpus},
                gpu_launches=int(launches_per_step * args.steps),
                roofline={"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                          "frac": achieved / peak, "traffic": traffic[0] if traffic else None,
                          "traffic_note": "bytes per launch, estimated: each layer's algorithmic bytes x the DRAM / algorithmic "
                                          "ratio of a single-launch ncu capture of its class (residual, block tail, "
                                          "pointwise, 3x3); the fc launch is not counted" if traffic else
                                          "no single-launch captures for this workload",
                          "frac_of_traffic": (traffic[1] / (tc_ms_step / 1e3) / 1e9 / peak) if traffic else None,
                          "frac_of_8TBs": achieved / HBM_NOMINAL_GBS,
                          "peak_source": peak_kind + " copy bandwidth",
                          "kernel": "igemm_i8_tc_kernel", "launches_per_step": n_tc,
                          "algorithmic_bytes_per_launch": total_bytes / n_tc,
                          "avg_launch_us": 1e3 * tc_ms_step / n_tc,
                          "tensor_tops": tensor_tops, "tensor_frac_of_4.5POPS": tensor_tops / INT8_PEAK_TOPS,
                          "share_of_step": tc_ms_step / ms_step})
    if c3_ms_step is not None:
        macs3 = sum(m for name, b, m, g in per_layer if g == 1 and name.endswith("b"))
        bytes3 = sum(b for name, b, m, g in per_layer if g == 1 and name.endswith("b"))
        n3 = sum(1 for name, b, m, g in per_layer if g == 1 and name.endswith("b"))
        tops3 = 2.0 * macs3 / (c3_ms_step / 1e3) / 1e12
        line["roofline_tensor"] = {"bound": "tensor", "kernel": "igemm_i8_tc_kernel, the %d 3x3 convolutions of a step" % n3,
                                   "achieved": tops3, "peak": INT8_PEAK_TOPS, "unit": "TOP/s", "frac": tops3 / INT8_PEAK_TOPS,
                                   "peak_source": "datasheet dense int8", "launches_per_step": n3,
                                   "avg_launch_us": 1e3 * c3_ms_step / n3,
                                   "hbm_frac_of_these_launches": bytes3 / (c3_ms_step / 1e3) / 1e9 / peak}
    if rank == 0 and not args.no_extras and world == 1:
        extra = {}
        try:
            with torch.cuda.stream(stream):
                # sustained: graph replays for about two seconds, median of 20-step blocks, own clock samples
                sampler = ClockSampler(_nvml_index(local_rank))
                sampler.start()
                t0 = time.perf_counter()
                blocks = []
                while time.perf_counter() - t0 < 2.0:
                    blocks.append(time_replays(torch, stream, g_full, 20, torch.cuda.synchronize))
                sclk = sampler.stop(t0, time.perf_counter())
                med = statistics.median(blocks)
                extra["sustained"] = {"seconds": round(time.perf_counter() - t0, 2), "blocks_of_20_steps": len(blocks),
                                      "ms_per_step_median": med, "ms_per_step_min": min(blocks), "ms_per_step_max": max(blocks),
                                      "value": batch / (med / 1e3), "unit": "images/s", "clocks": sclk}
                # the same step launched layer by layer without a CUDA graph
                for _ in range(2):
                    runner.forward(dev_images[0])
                torch.cuda.synchronize()
                g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                g0.record(stream)
                for _ in range(10):
                    runner.forward(dev_images[0])
                g1.record(stream)
                torch.cuda.synchronize()
                extra["eager_ms_per_step"] = g0.elapsed_time(g1) / 10
                ctx.sync()
            del g_full, g_body, g_tc, g_3x3, runner
            torch.cuda.empty_cache()
            others = [("mobilenet_v1", 32, None), ("mobilenet_v1", 256, None), ("resnet50", 1024, None)]
            if args.net != "resnet50":
                others = [("resnet50", 128, None)]
            for net, b, mb in others:
                key = "%s_b%d" % (net, b)
                extra[key] = measure_network(torch, plb, networks, ctx, stream, net, b, 10 if b <= 256 else 4, 3, mb)
            with torch.cuda.stream(stream):  # the layers' launches and the timing events on the ctx stream
                rows, vendor_tops = layer_table(plb, ctx)
            extra["layers"] = rows
            extra["int8_vendor_gemm_tops"] = vendor_tops
            line["roofline"]["tensor_frac_of_vendor_gemm"] = tensor_tops / vendor_tops
            if "roofline_tensor" in line:
                line["roofline_tensor"]["frac_of_vendor_gemm"] = line["roofline_tensor"]["achieved"] / vendor_tops
        except Exception as exc:  # the extras never cost the headline line
            extra["error"] = "%s: %s" % (type(exc).__name__, exc)
        line["extra"] = extra
    if rank == 0:
        if not args.no_cpu_baseline and args.gpus == 1:
            try:
                cpu_q = networks.build_quantized(spec, seed=1234, calib_images=4, device="cuda")
                # bounded sample: 16 images per host thread, about 10 s of CPU work
                sample = args.cpu_sample or 16 * max(os.cpu_count() or 1, 8)
                cb = cpu_baseline(cpu_q, spec, sample)
                cb.pop("seconds", None)
                line["cpu_baseline"] = cb
            except Exception as exc:  # the baseline is a reported number, never a reason to lose the line
                line["cpu_baseline"] = {"value": None, "unit": "images/s", "cores": os.cpu_count(),
                                        "kind": "unavailable", "sample": "failed: %s" % exc}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
