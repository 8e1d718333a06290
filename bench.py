#!/usr/bin/env python
"""Benchmark of the convolutional forward path: YOLOv3 608x608 images/s.

    python bench.py --gpus N --steps K --warmup W            this library on N B200s
    python bench.py --impl reference --steps K --warmup W    the reference's CPU path on the host cores
    python bench.py --impl reference-gpu [--ref-gpu-batch B] extra, never part of the default run: the reference's own CUDA
                                                             build (recompiled for sm_100a) through its network_predict,
                                                             stock and with this library attached (b200_attach[_network])

One step = one forward of one batch of synthetic images (seeded U[0,1) input,
seeded He-normal weights: no dataset or checkpoint is involved).  For N > 1 the
script is started by torchrun, one rank per GPU; every rank owns a full replica
of the weights (loaded once) and its own batch of images, there is no
collective on the data path; ranks meet only at the barriers around the timed
region, and the slowest rank's time is the job's time.

Prints ONE JSON line (rank 0).  `value` is the whole job's images/s with inputs
resident in HBM; `e2e` the same through the C ABI with pinned HOST buffers (H2D of
the batch and D2H of the three detection heads inside the timed region, two steps
in flight; `e2e.blocking_predict` is the blocking network_predict call);
`graph_replay` the device-resident forward as one CUDA graph per step; `roofline` describes the tensor-core convolution kernel, timed with
CUDA events between layers inside the timed region; `cpu_baseline` is the
unmodified reference (CPU build under oracle/_ref, else the CPU checker) timed
on a bounded sample on this box's host cores.  More keys: `strong` (N > 1: the same 64 images
split over the ranks, graph replay), `host_copy_ceiling` (plain pinned-memory copies of the step's bytes
on all ranks at once: what the host side can move, and `e2e` as a fraction of it), `other_configs`
(N = 1: ResNet-50 batch 256 and xnor Darknet-19 batch 128, value and roofline).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

UNIT = "images/s"

# DRAM traffic of the tensor-core convolution kernel as ncu measured it (dram__bytes_read.sum + dram__bytes_write.sum
# summed over the kernel's launches of one forward), as (bytes per image, bytes per forward independent of the batch:
# the weights, read once per launch).  Scaled by the images one step processes.
NCU_DRAM_TRAFFIC = {
    ("yolov3", "tf32", 608): (545_665_920.0, 247_579_648.0),
    ("conv3x3", "tf32", 224): (488.0e6 / 64, 0.0),
    ("conv1x1", "tf32", 224): (491.0e6 / 64, 0.0),
}


def workload_cfg(name: str, batch: int, size: int) -> tuple[str, str, str]:
    """(cfg text, metric name, description) of a benchmark workload.  `yolov3` is the headline; the others
    are the remaining benchmark configurations, reachable for profiling single kernels."""
    from darknet_b200 import synth
    if name == "yolov3":
        return synth.yolov3_cfg(batch, size), f"yolov3_{size}_forward_images_per_s", f"yolov3-{size} forward"
    if name == "yolov3-tiny":
        return synth.yolov3_tiny_cfg(batch, size), f"yolov3_tiny_{size}_forward_images_per_s", f"yolov3-tiny-{size} forward"
    if name == "resnet50":
        return synth.resnet50_cfg(batch, size), f"resnet50_{size}_forward_images_per_s", f"resnet50-{size} forward"
    if name == "darknet19-xnor":
        return synth.darknet19_cfg(batch, size, xnor=True), f"darknet19_xnor_{size}_forward_images_per_s", f"xnor darknet19-{size} forward"
    if name == "conv3x3":   # darknet53 mid-stage layer: 256 -> 512, 3x3, 52x52, batchnorm + leaky
        return synth.single_conv_cfg(batch, 256, 52, 52, 512, 3), "conv3x3_256_512_52_images_per_s", "isolated 3x3 conv 256->512 at 52x52"
    if name == "conv1x1":
        return synth.single_conv_cfg(batch, 512, 52, 52, 256, 1), "conv1x1_512_256_52_images_per_s", "isolated 1x1 conv 512->256 at 52x52"
    if name.startswith("block:"):   # block:C,HW: one residual block of darknet-53 (3x3 C->C, 1x1 C->C/2, 3x3 C/2->C, shortcut), for profiling
        c, hw = [int(t) for t in name[6:].split(",")]
        cfg = (synth._net(batch, hw, hw, c) + synth._conv(c, 3) + synth._conv(c // 2, 1) + synth._conv(c, 3) + synth._shortcut(-3))
        return cfg, f"block_{c}_{hw}_images_per_s", f"darknet-53 residual block, {c} channels at {hw}x{hw}"
    if name.startswith("conv:"):   # conv:C,HW,N,SIZE[,STRIDE]: any single layer, for profiling (batchnorm + leaky)
        v = [int(t) for t in name[5:].split(",")]
        c, hw, n, k = v[:4]
        st = v[4] if len(v) > 4 else 1
        return (synth.single_conv_cfg(batch, c, hw, hw, n, k, stride=st), f"conv{k}x{k}_{c}_{n}_{hw}_images_per_s",
                f"isolated {k}x{k}/{st} conv {c}->{n} at {hw}x{hw}")
    if name == "memlayers":   # maxpool / upsample / shortcut / route at the shapes of YOLOv3's 152x152 stage
        return synth.memory_layers_cfg(batch, 128, size or 152), "memory_layers_152_images_per_s", "maxpool, upsample, shortcut, route chained (128 channels, 152x152)"
    raise SystemExit(f"unknown workload {name}")


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "reference-gpu"])
    ap.add_argument("--ref-gpu-batch", type=int, default=0,
                    help="b200 arm: also time the reference's own CUDA build and the attach shim in a child process at this batch "
                         "(0, the default: skip); --impl reference-gpu: images per network_predict call (default 8)")
    ap.add_argument("--mode", default="tf32", choices=["tf32", "bf16"])
    ap.add_argument("--batch", type=int, default=64, help="images per GPU per step")
    ap.add_argument("--size", type=int, default=0, help="input width = height (default: 608 yolov3, 416 tiny, 224 classifiers)")
    ap.add_argument("--workload", default="yolov3",
                    help="yolov3 (the headline), yolov3-tiny, resnet50, darknet19-xnor, conv3x3, conv1x1, memlayers, conv:C,HW,N,SIZE[,STRIDE] "
                         "for one convolutional layer of that shape, or block:C,HW for one darknet-53 residual block")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="weak: --batch images on every GPU; strong: --batch images split over the GPUs")
    ap.add_argument("--cpu-sample", type=int, default=4, help="images of the CPU-baseline sample (0 = skip)")
    ap.add_argument("--layers", default="", help="write a per-layer time table to this file")
    ap.add_argument("--no-extras", action="store_true", help="skip the strong-scaling, copy-ceiling and other-configuration records")
    return ap.parse_args()


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_sustained": d["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """SM clock, power and throttle reasons sampled during the timed region: every 20 ms through NVML
    (read-only queries), or every 200 ms through nvidia-smi when NVML cannot be loaded."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, gpu_index: int):
        self.proc = None
        self.rows: list[tuple] = []     # (sm_mhz, max_mhz, watts, {reasons})
        self.stop_flag = False
        self.nvml = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.t = threading.Thread(target=self._poll, daemon=True)
            self.t.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _poll(self):
        n = self.nvml
        bits = {"hw_slowdown": getattr(n, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
                "hw_thermal_slowdown": getattr(n, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
                "sw_thermal_slowdown": getattr(n, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
                "sw_power_cap": getattr(n, "nvmlClocksThrottleReasonSwPowerCap", 0x4)}
        while not self.stop_flag:
            try:
                mhz = float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                watts = n.nvmlDeviceGetPowerUsage(self.handle) / 1000.0
                mask = int(n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                self.rows.append((mhz, self.max_mhz, watts, {k for k, b in bits.items() if mask & b}))
            except Exception:
                pass
            time.sleep(0.02)

    def _read(self):
        for line in self.proc.stdout:
            r = line.strip().split(", ")
            if len(r) >= 9:
                try:
                    self.rows.append((float(r[1]), float(r[2]), float(r[3]),
                                      {k for k, v in zip(self.NAMES, r[5:9]) if v.strip().lower().startswith("active")}))
                except ValueError:
                    pass

    def mark(self):
        return len(self.rows)

    def stop(self, start: int = 0):
        self.stop_flag = True
        if self.nvml is None and not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=3)
            except Exception:
                self.proc.kill()
        else:
            self.t.join(timeout=1)
        rows = self.rows[start:] or self.rows
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = sorted(r[0] for r in rows)
        reasons = set()
        for r in rows:
            reasons |= r[3]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": rows[0][1], "reasons": sorted(reasons),
                "power_w_max": max(r[2] for r in rows), "samples": len(rows),
                "source": "NVML, 20 ms" if self.nvml is not None else "nvidia-smi, 200 ms"}


def write_net_files(d: str, cfg: str, seed: int = 0):
    from darknet_b200 import synth
    params = synth.seeded_params(cfg, seed)
    with open(os.path.join(d, "net.cfg"), "w") as f:
        f.write(cfg)
    synth.write_weights(os.path.join(d, "net.weights"), params)
    return params


class CpuReference:
    """The reference's own CPU forward (network_predict, src/network.c:497-508) on `images` seeded
    images of YOLOv3, all host threads.  Uses oracle/_ref (the unmodified reference compiled from its
    own sources) when it was built, otherwise the CPU restatement."""

    def __init__(self, workload: str, size: int, images: int):
        from darknet_b200 import synth
        from oracle import network as orc
        self.images = images
        self.cfg, self.metric, self.desc = workload_cfg(workload, images, size)
        self.x = synth.seeded_input(self.cfg, 0)
        self.cores = os.cpu_count() or 1
        self.orc = orc
        with tempfile.TemporaryDirectory() as d:
            self.params = write_net_files(d, self.cfg)
            if orc.Reference.available():
                self.R = orc.Reference()
                devnull = os.open(os.devnull, os.O_WRONLY)
                saved = os.dup(2)
                os.dup2(devnull, 2)   # the reference prints its layer table to stderr
                try:
                    self.net = self.R.load(d + "/net.cfg", d + "/net.weights")
                finally:
                    os.dup2(saved, 2)
                    os.close(devnull)
                self.R.L.ref_set_threads(os.cpu_count() or 1)   # torchrun exports OMP_NUM_THREADS=1: use every host core
                self.cores = self.R.L.ref_max_threads()
                self.kind = "reference"
            else:
                self.R = None
                self.kind = "port"

    def seconds(self) -> float:
        """Wall-clock seconds of one forward of the sample."""
        if self.R is not None:
            return float(self.R.L.ref_time_predict(self.net, self.x.ctypes.data, 1))
        t0 = time.perf_counter()
        self.orc.forward_network(self.cfg, self.params, self.x)
        return time.perf_counter() - t0


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    images = 1
    ref = CpuReference(args.workload, args.size, images)
    times = []
    spent = 0.0
    for i in range(args.warmup + args.steps):
        sec = ref.seconds()
        spent += sec
        if i >= args.warmup:
            times.append(sec)
        if spent > 240 and times:   # keep the whole run within a few minutes
            break
    ms = 1000.0 * float(np.mean(times))
    value = images / (ms / 1000.0)
    line = {"impl": "reference", "metric": ref.metric, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": len(times), "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{ref.desc}, reference CPU path (stock -Ofast -fopenmp build), {images} image per step, "
                                   f"{ref.cores} host threads"},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": ref.cores, "kind": ref.kind,
                             "sample": f"{images} image(s) of {ref.desc} per step, network_predict on the host cores"},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def run_reference_gpu(args):
    """The unmodified reference's own CUDA path (im2col + cuBLAS + separate bias / batchnorm / activation
    kernels, its .cu files recompiled for sm_100a; oracle/_ref/libdarknet_ref_gpu.so) through its
    network_predict, host buffers in and out, on GPU 0.  A same-box row beside the CPU baseline; the
    reference allocates training buffers too, so it runs a smaller batch (its GEMMs are per image anyway)."""
    from darknet_b200 import synth
    from oracle import network as orc
    if not orc.ReferenceGpu.available():
        print(json.dumps({"impl": "reference-gpu", "unavailable": "oracle/_ref/libdarknet_ref_gpu.so was not built (make -C oracle refgpu)"}), flush=True)
        return
    batch = args.ref_gpu_batch if args.ref_gpu_batch > 0 else 8
    cfg, metric, desc = workload_cfg(args.workload, batch, args.size)
    d = tempfile.mkdtemp(prefix="dnb_refgpu_")
    write_net_files(d, cfg)
    ref = orc.ReferenceGpu()
    net = ref.load(os.path.join(d, "net.cfg"), os.path.join(d, "net.weights"))
    import torch
    # page-locked input for all three rows: network_predict pushes it with a blocking cudaMemcpy (src/cuda.c:153-158)
    x = torch.from_numpy(synth.seeded_input(cfg, 0, "normal" if args.workload.startswith("conv") else "uniform")).pin_memory().numpy()
    ref.time_predict(net, x, max(args.warmup, 1))
    sec = ref.time_predict(net, x, args.steps) / args.steps
    # the same `network` after b200_attach: Darknet's loop, buffers and layout, this library's kernels per layer
    import darknet_b200 as dn
    attached = ref.attach(net, dn.MODE_TF32)
    att = None
    if attached > 0:
        ref.time_predict(net, x, max(args.warmup, 1))
        asec = ref.time_predict(net, x, args.steps) / args.steps
        att = {"value": batch / asec, "unit": UNIT, "ms_per_step": asec * 1000.0, "layers_repointed": attached,
               "note": "forward_gpu pointers of the unmodified network re-pointed by b200_attach (TF32 plans, NCHW fp32 tensors at every layer boundary)"}
    # and with the whole forward pass handed over (b200_attach_network), still through Darknet's network_predict
    whole = None
    if attached > 0:
        ref.detach(net)
    if ref.attach_network(net, dn.MODE_TF32) > 0:
        ref.time_predict(net, x, max(args.warmup, 1))
        wsec = ref.time_predict(net, x, args.steps) / args.steps
        whole = {"value": batch / wsec, "unit": UNIT, "ms_per_step": wsec * 1000.0,
                 "note": "b200_attach_network: layer 0's forward_gpu runs the library's own network object, [yolo] and last-layer outputs copied into Darknet's buffers"}
    print(json.dumps({"impl": "reference-gpu", "metric": metric, "value": batch / sec, "unit": UNIT, "ms_per_step": sec * 1000.0, "attached": att,
                      "attached_network": whole,
                      "steps": args.steps, "dtype": "f32", "data": "synthetic",
                      "config": {"workload": f"{desc}, batch {batch}, the reference's CUDA build recompiled for sm_100a "
                                             "(im2col + cuBLAS sgemm per image), network_predict with host buffers"}}), flush=True)


def roofline_of(net, cfg: str, per_gpu: int, mean_ms, mode: str, workload: str, size: int):
    """Roofline object of a network's dominant kernel from per-layer CUDA-event times: the tensor-core convolution
    (FLOPs against the measured tensor peak, with its HBM-bound launches split out), the popcount convolution of an
    xnor network (word-popcounts per second), or the memory-bound layer kernels (bytes against the HBM copy rate).
    Returns (roofline, flops per layer, layer kinds, layer kernels)."""
    from darknet_b200 import synth
    kinds = [net.layer_type(i) for i in range(net.n)]
    kernels = [net.layer_kernel(i) for i in range(net.n)]
    flops = np.zeros(net.n)
    sections = synth.parse_cfg(cfg)[1:]
    shapes = {s.index: s for s in synth.conv_shapes(cfg)}
    for i, (k, opt) in enumerate(sections):
        if k == "convolutional":
            c, h, w = net.layer_shape(i)
            s = shapes[i]
            flops[i] = 2.0 * s.n * s.size * s.size * (s.c // s.groups) * h * w * per_gpu
    tc = np.array([kn.startswith("tc_") for kn in kernels])
    tc_ms = float(mean_ms[tc].sum())
    tc_flops = float(flops[tc].sum())
    peaks = load_peaks()
    achieved = tc_flops / (tc_ms / 1000.0) / 1e12 if tc_ms > 0 else 0.0
    # a kernel timed alone is held against the burst figure, one timed inside a long step against the sustained one
    alone = workload.startswith("conv")
    bf16_peak = peaks["bf16_tflops"] if alone else peaks["bf16_sustained"]
    peak = bf16_peak / (2.0 if mode == "tf32" else 1.0)
    big3 = np.array([bool(tc[i]) and sections[i][1].get("size") == "3" and shapes[i].c >= 64 for i in range(net.n)])
    big3_tflops = float(flops[big3].sum() / (mean_ms[big3].sum() / 1000.0) / 1e12) if big3.any() else None
    # the other launches of the same kernel (1x1 layers, 3x3 layers with fewer than 64 input channels) are bound by
    # HBM: algorithmic bytes = input + output of the layer in its storage type, the weights once, and the residual
    # a fused [shortcut] reads, over the same event durations
    es = 2.0 if mode == "bf16" else 4.0
    small = np.array([bool(tc[i]) and not big3[i] for i in range(net.n)])
    mem_bytes = 0.0
    for i in np.nonzero(small)[0]:
        c, h, w = net.layer_shape(int(i))
        stride = int(sections[i][1].get("stride", 1))
        sh = shapes[int(i)]
        mem_bytes += es * per_gpu * (sh.c * (h * stride) * (w * stride) + sh.n * h * w) + es * sh.n * sh.c * sh.size * sh.size
        if i + 1 < net.n and kinds[i + 1] == "shortcut" and mean_ms[i + 1] < 0.01:   # fused: its add is read by this launch
            mem_bytes += es * per_gpu * sh.n * h * w
    small_ms = float(mean_ms[small].sum())
    hbm_part = None
    if small.any() and small_ms > 0:
        gbs = mem_bytes / (small_ms / 1000.0) / 1e9
        hbm_part = {"launches_per_step": int(small.sum()), "ms_per_step": small_ms, "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": gbs / peaks["hbm_gbs"], "what": "1x1 layers and 3x3 layers with fewer than 64 input channels: HBM-bound launches of the same kernel"}
    roofline = {"kernel": "conv_tc_kernel", "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak,
                "traffic": (lambda t: None if t is None else t[0] * per_gpu + t[1])(NCU_DRAM_TRAFFIC.get((workload, mode, size))),
                "traffic_unit": "bytes per step per GPU (ncu dram read+write of all launches of this kernel)",
                "launches_per_step": int(tc.sum()), "avg_launch_ms": tc_ms / max(int(tc.sum()), 1),
                "share_of_step": tc_ms / float(mean_ms.sum()),
                "peak_source": f"{peaks['source']}: cuBLAS bf16 {'burst' if alone else 'sustained'} {bf16_peak} TFLOP/s"
                               + (" / 2 (TF32 runs at half the BF16 tensor rate)" if mode == "tf32" else ""),
                "conv3x3_c64plus_tflops": big3_tflops,
                "conv3x3_c64plus_frac": (big3_tflops / peak) if big3_tflops else None,
                "hbm_bound_launches": hbm_part}

    if not tc.any():
        # a network of memory-bound layers only: algorithmic bytes per layer (4*(in+out) for maxpool and upsample,
        # 12 B per element for shortcut, 8 B per element for route) over the event time, against the HBM copy rate
        es_m = 2.0 if mode == "bf16" else 4.0
        total_b, per_layer = 0.0, []
        net_opt = synth.parse_cfg(cfg)[0][1]
        prev = (int(net_opt["channels"]), int(net_opt["height"]), int(net_opt["width"]))
        for i in range(net.n):
            c, h, w = net.layer_shape(i)
            out_e = per_gpu * c * h * w
            in_e = per_gpu * prev[0] * prev[1] * prev[2]
            b = {"maxpool": es_m * (in_e + out_e), "upsample": es_m * (in_e + out_e), "shortcut": 3 * es_m * out_e, "route": 2 * es_m * out_e}.get(kinds[i], 0.0)
            per_layer.append({"layer": i, "kind": kinds[i], "GB": b / 1e9, "ms": float(mean_ms[i]), "GBps": b / (mean_ms[i] / 1000.0) / 1e9 if mean_ms[i] > 0 else None})
            total_b += b
            prev = (c, h, w)
        gbs = total_b / (float(mean_ms.sum()) / 1000.0) / 1e9
        roofline = {"kernel": "maxpool / upsample / shortcut / route kernels", "bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": gbs / peaks["hbm_gbs"], "traffic": None, "per_layer": per_layer,
                    "peak_source": f"{peaks['source']}: STREAM-style copy"}

    xn = np.array([kn.startswith("xnor") for kn in kernels])
    if xn.any() and float(mean_ms[xn].sum()) > float(mean_ms[tc].sum()):
        # an xnor network: the popcount convolution dominates.  Work = one 32-bit xnor + popcount per 32 input channels
        # per tap per filter per output pixel; no published peak exists for it, the fraction is against the integer
        # pipe's popc issue rate (16 per SM per clock at the sampled clock is the figure NVIDIA documents for sm_100)
        words = 0.0
        for i in np.nonzero(xn)[0]:
            c, h, w = net.layer_shape(int(i))
            sh = shapes[int(i)]
            words += float(per_gpu) * sh.n * sh.size * sh.size * ((sh.c + 31) // 32) * h * w
        x_ms = float(mean_ms[xn].sum())
        rate = words / (x_ms / 1000.0) / 1e12
        if any(kn == "xnor_tc" for kn in kernels):
            # int8 sign tensors through the tensor cores (kind::i8): the integer sums cost a few per cent of the int8 tensor
            # rate; what bounds the layer is the fp32 activations around it.  Algorithmic bytes per layer: fp32 input read
            # once by the sign pass, int8 signs written and read once, fp32 output written, the int8 weights once.
            # Where one xnor layer feeds the next, the first writes the second's signs from its epilogue (1 byte per output
            # more) and the second reads only those.
            bytes_ = 0.0
            passes = 0
            for i in np.nonzero(xn)[0]:
                c, h, w = net.layer_shape(int(i))
                sh = shapes[int(i)]
                stride = int(sections[int(i)][1].get("stride", 1))
                in_e = float(per_gpu) * sh.c * (h * stride) * (w * stride)
                out_e = float(per_gpu) * sh.n * h * w
                desc = net.layer_describe(int(i))
                given, gives = "signs_in=1" in desc, "signs_out=1" in desc
                passes += 0 if given else 1
                bytes_ += (1.0 * in_e if given else 4.0 * in_e + 2.0 * in_e) + (5.0 if gives else 4.0) * out_e + sh.n * sh.c * sh.size * sh.size
            gbs = bytes_ / (x_ms / 1000.0) / 1e9
            ops = 2.0 * 32.0 * words   # multiply-adds of +-1 values, two operations each
            roofline = {"kernel": "conv_tc_kernel (int8 kind) + pack_sign_i8_kernel", "bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                        "frac": gbs / peaks["hbm_gbs"], "traffic": None, "launches_per_step": int(xn.sum()) + passes, "ms_per_step": x_ms,
                        "share_of_step": x_ms / float(mean_ms.sum()), "integer_tops": ops / (x_ms / 1000.0) / 1e12,
                        "peak_source": f"{peaks['source']}: STREAM-style copy",
                        "what": "xnor layers as int8 sign tensors on tcgen05 (exact int32 sums); bytes = fp32 output + int8 weights + either the fp32 input and its int8 signs written and read (sign pass) or the int8 signs the previous xnor layer wrote (1 byte written there, 1 read here)"}
        else:
            roofline = {"kernel": "conv_xnor_kernel", "bound": "popc issue", "achieved": rate, "unit": "T word-popcounts/s", "peak": None, "frac": None,
                        "binary_tops": rate * 64.0, "traffic": None, "launches_per_step": int(xn.sum()), "ms_per_step": x_ms,
                        "share_of_step": x_ms / float(mean_ms.sum()),
                        "what": "bit-packed xnor + popcount GEMM on the integer pipe; binary_tops counts 2 x 32 binary operations per word"}
    return roofline, flops, kinds, kernels


def side_config(workload: str, batch: int, size: int, mode_name: str, steps: int):
    """Device-resident forward of another benchmark configuration on the current GPU: images/s from CUDA events
    around `steps` forwards after three warm-ups, and the roofline object of its dominant kernel."""
    import torch

    import darknet_b200 as dn
    from darknet_b200 import synth
    cfg, metric, desc = workload_cfg(workload, batch, size)
    d = tempfile.mkdtemp(prefix="dnb_side_")
    write_net_files(d, cfg)
    net = dn.Network(cfg, os.path.join(d, "net.weights"), dn.MODE_TF32 if mode_name == "tf32" else dn.MODE_BF16, text=True)
    x_dev = torch.from_numpy(synth.seeded_input(cfg, 0, "uniform")).cuda()
    stream = torch.cuda.current_stream()
    for _ in range(3):
        net.forward(x_dev)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for k in range(steps):
        net.forward_timed(x_dev, slot=k)
    e1.record(stream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    mean_ms = np.stack([net.timed_ms(k) for k in range(steps)]).astype(np.float64).mean(axis=0)
    roofline, flops, _, _ = roofline_of(net, cfg, batch, mean_ms, mode_name, workload, size)
    rec = {"metric": metric, "value": batch / (ms / 1000.0), "unit": UNIT, "ms_per_step": ms, "steps": steps, "dtype": mode_name,
           "config": {"workload": f"{desc}, batch {batch}, device-resident"}, "gpu_launches": net.launches * steps,
           "tflops_algorithmic": float(flops.sum()) / (ms / 1000.0) / 1e12, "roofline": roofline}
    net.close()
    return rec


def run_b200(args):
    import torch
    import torch.distributed as dist

    import darknet_b200 as dn
    from darknet_b200 import synth

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs CUDA devices; there is no CPU fallback"
    torch.cuda.set_device(local)
    dn.check(dn.lib().dnb_set_device(local))
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from darknet_b200.shard import bind_near_gpu, max_over_ranks, shard_batch
    # several ranks share the host: each keeps its threads and its pinned buffers in the memory next to its GPU
    near_cpus = bind_near_gpu(local) if world > 1 and not os.environ.get("DNB_NO_NUMA_BIND") else []
    # weak: every rank forwards --batch images; strong: --batch images are cut into contiguous slices
    per_gpu = args.batch if args.scaling == "weak" else max(1, shard_batch(args.batch, world, rank)[1])
    mode = dn.MODE_TF32 if args.mode == "tf32" else dn.MODE_BF16

    sampler = ClockSampler(local) if rank == 0 else None
    cfg, metric, desc = workload_cfg(args.workload, per_gpu, args.size)
    # weights: written once by rank 0, every rank loads the same file into its own HBM
    wdir = os.path.join(tempfile.gettempdir(), f"dnb_bench_{os.environ.get('MASTER_PORT', 'single')}_{args.workload}_{args.size}")
    if rank == 0:
        os.makedirs(wdir, exist_ok=True)
        write_net_files(wdir, cfg)
    if world > 1:
        dist.barrier()
    net = dn.Network(cfg, os.path.join(wdir, "net.weights"), mode, text=True)
    x_host = torch.from_numpy(synth.seeded_input(cfg, rank, "normal" if args.workload.startswith(("conv", "block")) else "uniform")).pin_memory()
    x_dev = x_host.cuda()
    stream = torch.cuda.current_stream()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident forward
    for _ in range(max(args.warmup, 3)):
        net.forward(x_dev)
    barrier()
    mark = sampler.mark() if sampler else 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for s in range(args.steps):
        net.forward_timed(x_dev, slot=s)
    e1.record(stream)
    barrier()
    ms_total = e0.elapsed_time(e1)
    layer_ms = np.stack([net.timed_ms(s) for s in range(args.steps)]).astype(np.float64)   # [steps, layers]
    ms_step = max_over_ranks(ms_total, "cuda") / args.steps
    clocks = sampler.stop(mark) if sampler else None
    total_images = per_gpu * world if args.scaling == "weak" else args.batch
    value = total_images / (ms_step / 1000.0)

    # ---- the same forward replayed as one CUDA graph (no per-layer events): what a caller gets from
    # dnb_network_enable_graph; matters at small batches, where the launches outweigh the kernels
    gstream = torch.cuda.Stream()
    net.enable_graph(True)
    for _ in range(3):                                   # eager, capture, first replay
        net.forward(x_dev, stream=gstream.cuda_stream)
    gstream.synchronize()
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g0.record(gstream)
    for _ in range(args.steps):
        net.forward(x_dev, stream=gstream.cuda_stream)
    g1.record(gstream)
    gstream.synchronize()
    graph_ms_step = max_over_ranks(g0.elapsed_time(g1), "cuda") / args.steps
    net.enable_graph(False)

    # ---- end to end with HOST buffers.  Every step uploads its own images from pinned host memory and
    # its results are read on the host.  Two ways of calling: the blocking network_predict, and the same
    # split into submit/collect with two steps in flight (a caller streaming batches), where the copies of
    # one step overlap the layers of the next.  The second is the headline; both are reported.
    x_host2 = x_host.clone().pin_memory()
    for _ in range(2):
        net.predict(x_host)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        out = net.predict(x_host)
        float(out[0, 0])   # the result is read on the host
    torch.cuda.synchronize()
    sync_ms = (time.perf_counter() - t0) * 1000.0
    sync_ms_step = max_over_ranks(sync_ms, "cuda") / args.steps
    hosts = [x_host, x_host2]
    for k in range(2):
        net.submit(hosts[k])
    for k in range(2):
        net.collect()
    barrier()
    t0 = time.perf_counter()
    net.submit(hosts[0])
    for k in range(1, args.steps):
        net.submit(hosts[k & 1])
        float(net.collect()[0, 0])
    float(net.collect()[0, 0])
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1000.0
    e2e_ms_step = max_over_ranks(e2e_ms, "cuda") / args.steps
    kinds = [net.layer_type(i) for i in range(net.n)]
    act_gb = sum(4.0 * per_gpu * int(np.prod(net.layer_shape(i))) for i in range(net.n)) / 1e9
    d2h_last = 0 if kinds[-1] == "yolo" else 4 * per_gpu * net.outputs
    d2h = d2h_last + sum(4 * per_gpu * int(np.prod(net.layer_shape(i))) for i, k in enumerate(kinds) if k == "yolo")
    h2d = 4 * per_gpu * net.inputs
    mean_ms = layer_ms.mean(axis=0)
    launches_per_step = net.launches
    extras = not args.no_extras and args.workload == "yolov3" and args.scaling == "weak"

    # ---- what the host side can move: every rank copies one step's bytes (its images up, its head outputs down) between
    # the same kind of pinned buffers and its GPU, all ranks at once, upload and download on their own streams, plain
    # asynchronous copies and nothing else.  `e2e` can at best reach this.
    copy_ceiling = None
    if extras:
        up, down = torch.cuda.Stream(), torch.cuda.Stream()
        dev_out = torch.empty(max(d2h // 4, 1), dtype=torch.float32, device="cuda")
        host_out = torch.empty(max(d2h // 4, 1), dtype=torch.float32).pin_memory()
        dev_in = torch.empty_like(x_dev)

        def copy_steps(k):
            for _ in range(k):
                with torch.cuda.stream(up):
                    dev_in.copy_(x_host, non_blocking=True)
                with torch.cuda.stream(down):
                    host_out.copy_(dev_out, non_blocking=True)
            up.synchronize()
            down.synchronize()

        copy_steps(2)
        barrier()
        t0 = time.perf_counter()
        copy_steps(args.steps)
        copy_ms_step = max_over_ranks((time.perf_counter() - t0) * 1000.0, "cuda") / args.steps
        agg = (h2d + d2h) * world / (copy_ms_step / 1000.0) / 1e9
        copy_ceiling = {"ms_per_step": copy_ms_step, "aggregate_gb_per_s": agg, "per_gpu_gb_per_s": agg / world,
                        "images_per_s": total_images / (copy_ms_step / 1000.0),
                        "e2e_fraction": copy_ms_step / e2e_ms_step,
                        "what": f"{world} rank(s) at once: {h2d / 1e6:.0f} MB up and {d2h / 1e6:.0f} MB down per rank per step, pinned memory, one "
                                "asynchronous copy each way on separate streams, no kernels; e2e_fraction = this time / the e2e step time"}
        del dev_out, host_out, dev_in

    # ---- strong scaling, the benchmark configuration's own split: --batch images cut into one contiguous slice per
    # rank (replicated weights, no collective), the device-resident forward replayed as a CUDA graph
    strong = None
    if extras and world > 1:
        s_per = shard_batch(args.batch, world, rank)[1]
        s_cfg = workload_cfg(args.workload, s_per, args.size)[0]
        s_net = dn.Network(s_cfg, os.path.join(wdir, "net.weights"), mode, text=True)
        sx = x_dev[:s_per].contiguous()
        s_net.enable_graph(True)
        for _ in range(4):
            s_net.forward(sx, stream=gstream.cuda_stream)
        gstream.synchronize()
        barrier()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record(gstream)
        for _ in range(args.steps):
            s_net.forward(sx, stream=gstream.cuda_stream)
        s1.record(gstream)
        gstream.synchronize()
        strong_ms = max_over_ranks(s0.elapsed_time(s1), "cuda") / args.steps
        one_gpu = per_gpu / (graph_ms_step / 1000.0)          # a whole batch on one GPU, same replay, same run
        strong = {"images_per_step": args.batch, "images_per_gpu": s_per, "ms_per_step": strong_ms, "value": args.batch / (strong_ms / 1000.0),
                  "unit": UNIT, "one_gpu_value": one_gpu, "speedup": (args.batch / (strong_ms / 1000.0)) / one_gpu,
                  "efficiency": (args.batch / (strong_ms / 1000.0)) / one_gpu / world,
                  "what": f"{args.batch} images split over {world} GPUs, device-resident forward as one CUDA graph per rank, max over ranks; "
                          "one_gpu_value is the same batch on one GPU measured in this run"}
        s_net.close()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    roofline, flops, kinds, kernels = roofline_of(net, cfg, per_gpu, mean_ms, args.mode, args.workload, args.size)

    if args.layers:
        with open(args.layers, "w") as f:
            f.write("layer kind kernel out_c out_h out_w ms gflop tflops\n")
            for i in range(net.n):
                c, h, w = net.layer_shape(i)
                f.write(f"{i} {kinds[i]} {kernels[i]} {c} {h} {w} {mean_ms[i]:.4f} {flops[i] / 1e9:.2f} "
                        f"{(flops[i] / (mean_ms[i] / 1000.0) / 1e12) if mean_ms[i] > 0 else 0:.1f}\n")

    # ---- the other benchmark configurations that fit one GPU, device-resident (N = 1 only)
    other = None
    if extras and world == 1:
        net.close()
        del x_dev
        torch.cuda.empty_cache()
        other = {}
        for name, batch, o_mode in (("resnet50", 256, args.mode), ("darknet19-xnor", 128, "tf32")):
            try:
                other[name] = side_config(name, batch, 224, o_mode, max(args.steps, 5))
            except Exception as e:   # noqa: BLE001
                other[name] = {"unavailable": repr(e)[:300]}

    cpu = None
    if args.cpu_sample > 0:
        n_cpu = args.cpu_sample if world == 1 else 1    # rank 0's host cores are shared with the other ranks' processes by then idle
        args.cpu_sample = n_cpu
        ref = CpuReference(args.workload, args.size, args.cpu_sample)
        ref.seconds()   # first touch of the reference's freshly allocated buffers
        sec = ref.seconds()
        cpu = {"value": args.cpu_sample / sec, "unit": UNIT, "cores": ref.cores, "kind": ref.kind,
               "sample": f"{args.cpu_sample} image(s) of {desc}, second of two network_predict calls on the host cores ({sec:.1f} s)"}

    # the reference's own GPU path on the same box, in a child process (it exits on any error and holds tens of GB)
    ref_gpu = None
    if world == 1 and args.ref_gpu_batch > 0 and not args.workload.startswith("conv"):
        try:
            p = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference-gpu", "--workload", args.workload,
                                "--size", str(args.size), "--ref-gpu-batch", str(args.ref_gpu_batch), "--steps", "3", "--warmup", "1"],
                               capture_output=True, text=True, timeout=600)
            rows = [ln for ln in p.stdout.splitlines() if ln.startswith("{")]
            ref_gpu = json.loads(rows[-1]) if rows else {"unavailable": f"child exited {p.returncode}: {p.stderr[-200:]}"}
        except Exception as e:   # noqa: BLE001
            ref_gpu = {"unavailable": repr(e)[:200]}

    line = {"metric": metric, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
            "dtype": args.mode, "data": "synthetic",
            "config": {"workload": f"{desc}, batch {per_gpu} per GPU ({total_images} images per step over {world} GPU)",
                       "global_batch": total_images, "parallelism": f"dp{world} (image sharding, replicated weights, no collective)",
                       "host_binding": f"rank 0 bound to {len(near_cpus)} CPUs next to its GPU" if near_cpus else "none",
                       "l2": f"inputs larger than L2: every step streams {act_gb:.1f} GB of layer outputs through HBM, no flush needed",
                       "tflops_algorithmic": float(flops.sum()) * world / (ms_step / 1000.0) / 1e12},
            "e2e": {"value": total_images / (e2e_ms_step / 1000.0), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms_step, "timer": "host wall clock around K submit/collect steps, two in flight",
                    "blocking_predict": {"value": total_images / (sync_ms_step / 1000.0), "ms_per_step": sync_ms_step}},
            "graph_replay": {"value": total_images / (graph_ms_step / 1000.0), "unit": UNIT, "ms_per_step": graph_ms_step,
                             "what": "the device-resident forward as one CUDA graph launch per step (dnb_network_enable_graph)"},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu, "reference_gpu": ref_gpu,
            "strong": strong, "host_copy_ceiling": copy_ceiling, "other_configs": other}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    if not args.size:
        args.size = {"yolov3": 608, "yolov3-tiny": 416, "memlayers": 152}.get(args.workload, 224)
    if args.impl == "reference":
        run_reference(args)
    elif args.impl == "reference-gpu":
        run_reference_gpu(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
