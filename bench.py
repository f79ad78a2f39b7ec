#!/usr/bin/env python
"""Benchmark of the sparse 3D front end (voxelise -> 14 sparse conv layers -> dense BEV, fp16).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload sweep|single|voxelize|subm16]

One process per GPU (torchrun sets RANK / LOCAL_RANK / WORLD_SIZE for N > 1). A step is one pass over
the rank's shard of frames (default: 512 synthetic 120,000-point frames per GPU, the throughput-sweep
configuration). Frames are independent, so ranks exchange nothing on the data path; the process group
only carries the barrier and the max-over-ranks of the device time. Rank 0 prints one JSON line.

--impl reference times the CPU restatement of the reference plugins (oracle/, all host threads) on a
bounded sample of the same frames: the reference itself has no CPU implementation and cannot be built
without TensorRT.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
METRIC = "frames/sec (voxelize + sparse 3D backbone + dense BEV, fp16)"


def load_package():
    name = "se_ssd_ai_trt_b200"
    if name in sys.modules:
        return sys.modules[name]
    path = os.path.join(ROOT, "se-ssd-ai-trt_b200", "__init__.py")
    spec = importlib.util.spec_from_file_location(name, path, submodule_search_locations=[os.path.dirname(path)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def measured_traffic(workload, kernel):
    """DRAM bytes per frame and launch of `kernel` (dram__bytes_read.sum + dram__bytes_write.sum averaged over its
    launches) from the committed record of an ncu capture, with where that record comes from; (None, None) when
    there is no record for this workload and kernel. Traffic grows in proportion to the frames of a launch."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    try:
        with open(path) as f:
            rec = json.load(f)
    except (OSError, ValueError):
        return None, None
    k = rec.get("workloads", {}).get(workload, {}).get(kernel)
    if not k:
        return None, None
    src = "ncu capture of a %d-frame launch scaled by frames per launch; %s at commit %s" % (
        rec.get("frames_per_launch", 0), rec.get("command", "?"), rec.get("commit", "?"))
    return float(k["dram_bytes_per_frame"]), src


def measured_l2_to_sm(workload, kernel):
    """L2 -> SM bytes per frame of one launch of `kernel` from the same record (the gathers re-read every input row
    once per kernel offset that reaches it), or None. Captured for one launch of the 1/4-resolution layers."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    try:
        with open(path) as f:
            rec = json.load(f)
    except (OSError, ValueError):
        return None
    k = rec.get("workloads", {}).get(workload, {}).get(kernel) or {}
    v = k.get("l2_to_sm_bytes_per_frame_quarter_resolution_launch")
    return float(v) if v else None

WORKLOADS = {
    # name: (points per frame, object clusters, frames per GPU per step, max_voxels, frames per launch group)
    "sweep": dict(points=120000, boxes=40, frames=512, max_voxels=200000, batch=32, streams=2,
                  desc="throughput sweep: 512 frames x 120,000 points per GPU"),
    "single": dict(points=20000, boxes=15, frames=2048, max_voxels=60000, batch=32,
                   desc="20,000-point frames (single-frame backbone case), 2048 per GPU"),
    # the two small cases have their own timing loops (run_voxelize, run_subm16)
    "voxelize": dict(points=20000, boxes=15, frames=2048, max_voxels=20000, batch=64,
                     desc="voxelisation alone: 20,000-point frames, max 20,000 voxels, 5 points per voxel"),
    "subm16": dict(points=0, boxes=0, frames=1, max_voxels=20000, batch=1,
                   desc="one SubMConv3d 16->16, 3x3x3, fp32, batch 1, 16,000 active voxels in [41,1600,1408]"),
}


def make_frames(pkg, wl, nframes, first_index, threads=8):
    """Seeded synthetic frames [nframes, P, 4] (+ sizes); stands in for the reference's KITTI loop."""
    P = wl["points"]
    out = np.empty((nframes, P, 4), np.float32)

    def work(lo, hi):
        for f in range(lo, hi):
            seed = pkg.sharding.frame_seed(first_index + f)
            out[f] = pkg.synth.lidar_frame(seed, n_points=P, n_boxes=wl["boxes"])

    step = (nframes + threads - 1) // threads
    ts = [threading.Thread(target=work, args=(i, min(nframes, i + step))) for i in range(0, nframes, step)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    return out, np.full(nframes, P, np.int32)


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of one GPU while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def stop(self, t_begin=None, t_end=None):
        """Summary of the samples taken in [t_begin, t_end] (the timed region; nvidia-smi needs a second to
        start, so the sampler is started before the warm-up passes)."""
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        lines = [ln for ts, ln in self.lines if t_begin is None or t_begin <= ts <= t_end + 0.25]
        if not lines and self.lines and t_begin is not None:
            # a timed region shorter than the sampling period: take the two samples nearest to it
            mid = 0.5 * (t_begin + t_end)
            lines = [ln for _, ln in sorted(self.lines, key=lambda x: abs(x[0] - mid))[:2]]
        for ln in lines:
            p = [t.strip() for t in ln.split(",")]
            if len(p) < 8:
                continue
            try:
                sm.append(float(p[0]))
                mx.append(float(p[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm=float(p["hbm_gbs"]), tensor=float(p["bf16_tflops"]),
                    tensor_sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), source="measured")
    return dict(hbm=6650.0, tensor=1590.0, tensor_sustained=1400.0, source="fallback")


def layer_costs(pkg, rows_in, rows_out, pairs, esize=2):
    """Algorithmic bytes and flops per conv layer for one frame set: bytes = input rows x Cin + output rows x Cout
    + the weights (all fp16) + 16 B of coordinates per input row (and per output row of a strided layer);
    flops = 2 x rulebook pairs x Cin x Cout."""
    out = []
    for l, ni, no, p in zip(pkg.schedule.LAYERS, rows_in, rows_out, pairs):
        b = ni * l.cin * esize + no * l.cout * esize + l.kvol * l.cin * l.cout * esize + 16 * ni
        if not l.subm:
            b += 16 * no + 4
        out.append(dict(name=l.name, bytes=float(b), flops=2.0 * p * l.cin * l.cout))
    return out


def cpu_baseline(pkg, wl, frames, sizes, seconds_hint=20.0):
    """Times the CPU oracle (all host threads) on a bounded sample of the same frames."""
    sys.path.insert(0, ROOT)
    from oracle import binding as oracle

    threads = oracle.hardware_threads() or os.cpu_count() or 1
    per_frame = 5.5 * wl["points"] / 120000.0      # single-thread seconds per frame, measured once offline
    n = int(max(threads, min(len(frames), round(seconds_hint / per_frame * threads))))
    n = min(n, len(frames))
    w, sc, sh = pkg.random_weights()
    sec, status = oracle.front_end_frames(frames[:n], sizes[:n], pkg.synth.POINT_RANGE, pkg.synth.VOXEL_SIZE,
                                          wl["max_voxels"], pkg.schedule.LAYERS,
                                          np.concatenate([t.ravel() for t in w]), np.concatenate(sc),
                                          np.concatenate(sh), fp16=True, nthreads=threads, with_dense=True)
    return dict(value=n / sec, unit="frames/s", cores=threads, kind="port",
                sample=f"{n} of the step's frames, {threads} host threads, fp16-storage emulation, {sec:.1f} s",
                status=status), n, sec


def run_reference(args, pkg, wl, rank, world):
    """--impl reference: the CPU restatement of the reference plugins, timed on the host cores."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    per_step = max(threads, 8)
    frames, sizes = make_frames(pkg, wl, min(wl["frames"], per_step), 0)
    total_s, total_f, info = 0.0, 0, None
    for step in range(args.warmup + args.steps):
        info, n, sec = cpu_baseline(pkg, wl, frames, sizes, seconds_hint=1e-9)
        if step >= args.warmup:
            total_s += sec
            total_f += n
        if step == 0 and sec * (args.warmup + args.steps) > 240:   # keep the whole run within minutes
            args.steps = max(1, int(240 / sec) - args.warmup)
            if step >= args.warmup + args.steps:
                break
    value = total_f / total_s if total_s > 0 else info["value"]
    info["value"] = value
    line = dict(impl="reference", metric=METRIC, value=value, unit="frames/s", n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=1000.0 * total_s / max(args.steps, 1), higher_is_better=True,
                scaling="weak", vs_baseline=None, dtype="f16", data="synthetic",
                config=dict(workload=args.workload, description=wl["desc"], points_per_frame=wl["points"],
                            frames_per_gpu_per_step=wl["frames"], max_voxels=wl["max_voxels"],
                            sample_frames_per_step=total_f // max(args.steps, 1),
                            parallelism="host threads of rank 0, one frame per thread"),
                cpu_baseline=info,
                e2e=dict(value=value, unit="frames/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line), flush=True)


def _clocked(fn, steps, warmup, sampler_index=0):
    """fn() enqueues one step on the current stream; returns (ms per step, clocks summary)."""
    import torch

    sampler = ClockSampler(sampler_index)
    sampler.start()
    for _ in range(max(warmup, 3)):
        fn()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    ev0.record()
    for _ in range(steps):
        fn()
    ev1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop(t0, time.perf_counter())
    return ev0.elapsed_time(ev1) / steps, clocks


def run_voxelize(args, pkg, wl):
    """Voxelisation alone (20,000-point frames, 20,000 voxels max, mean of up to 5 points): frames/s and
    algorithmic GB/s (16 B per point read, 28 B per voxel written, fp32 features)."""
    import torch

    F, P, B = wl["frames"], wl["points"], wl["batch"]
    frames, sizes = make_frames(pkg, wl, F, 0)
    d_pts, d_sizes = torch.from_numpy(frames).cuda(), torch.from_numpy(sizes).cuda()
    params = pkg.voxel_params(wl["max_voxels"])
    outs = [pkg.voxelize(d_pts[i:i + B], d_sizes[i:i + B], params) for i in range(0, F, B)][:1]   # shapes + status
    assert outs[0]["status"] & ~pkg.STATUS_VOXEL_OVERFLOW == 0
    ws = torch.empty(pkg.lib().sessd_voxelize_workspace_bytes(__import__("ctypes").byref(params), B, P), dtype=torch.uint8,
                     device="cuda")
    vox = torch.empty((B, wl["max_voxels"], 4), device="cuda")
    coors = torch.empty((B, wl["max_voxels"], 4), dtype=torch.int32, device="cuda")
    num = torch.empty((B,), dtype=torch.int32, device="cuda")

    def step():
        for i in range(0, F, B):
            pkg.voxelize_into(d_pts[i:i + B], d_sizes[i:i + B], params, vox, coors, num, ws)

    launches0 = pkg.launch_count()
    ms, clocks = _clocked(step, args.steps, args.warmup)
    launches = (pkg.launch_count() - launches0) // (args.steps + max(args.warmup, 3))
    voxels = 0
    for i in range(0, F, B):
        pkg.voxelize_into(d_pts[i:i + B], d_sizes[i:i + B], params, vox, coors, num, ws)
        voxels += int(num.sum())
    byts = 16.0 * F * P + voxels * 28.0 + 4.0 * F
    pk = peaks()
    ach = byts / (ms / 1e3) / 1e9
    # CPU: the oracle's voxeliser, one thread, on a bounded sample
    sys.path.insert(0, ROOT)
    from oracle import binding as oracle
    n_cpu = 64
    t0 = time.perf_counter()
    for f in range(n_cpu):
        oracle.voxelize(frames[f], pkg.synth.POINT_RANGE, pkg.synth.VOXEL_SIZE, wl["max_voxels"])
    cpu_s = time.perf_counter() - t0
    return dict(metric="frames/sec (voxelization alone)", value=F / (ms / 1e3), unit="frames/s", n_gpus=1, steps=args.steps,
                warmup=max(args.warmup, 3), ms_per_step=ms, higher_is_better=True, scaling="weak", vs_baseline=None,
                dtype="f32", data="synthetic",
                config=dict(workload="voxelize", description=wl["desc"], points_per_frame=P, frames_per_step=F,
                            frames_per_call=B, max_voxels=wl["max_voxels"], voxels_per_frame=voxels / F,
                            l2="inputs larger than L2 (points of one step: %.0f MB)" % (F * P * 16 / 1e6)),
                gpu_launches=int(launches * args.steps), clocks=clocks,
                roofline=dict(bound="hbm", achieved=ach, peak=pk["hbm"], unit="GB/s", frac=ach / pk["hbm"], traffic=None,
                              kernel="voxel_insert + count/emit (whole call)", peak_source=pk["source"]),
                cpu_baseline=dict(value=n_cpu / cpu_s, unit="frames/s", cores=1, kind="port",
                                  sample=f"{n_cpu} of the step's frames, one host thread, {cpu_s:.1f} s"))


def run_subm16(args, pkg, wl):
    """One SubMConv3d 16->16, 3x3x3, fp32, batch 1 on 16,000 active voxels (rulebook + contraction, one plugin call):
    microseconds per call, pair flops and algorithmic bytes per second."""
    import torch

    S = pkg.synth
    coors_np = S.active_voxels()
    n = len(coors_np)
    feat_np = S.normal_f32(S.SEED_BASE + 11, (n, 16))
    W = S.normal_f32(S.SEED_BASE + 12, (27, 16, 16), 1.0 / np.sqrt(27 * 16))
    layer = pkg.schedule.ConvLayer("subm", True, 16, 16, (3, 3, 3), (1, 1, 1), (1, 1, 1), (41, 1600, 1408), (41, 1600, 1408))
    maxV = wl["max_voxels"]
    p = pkg.conv_params(layer, maxV)
    w = pkg.ConvWeights(p, W, None, None, False, pkg.F32)
    feat = torch.zeros((1, maxV, 16), device="cuda")
    coors = torch.zeros((1, maxV, 4), dtype=torch.int32, device="cuda")
    feat[0, :n] = torch.from_numpy(feat_np).cuda()
    coors[0, :n] = torch.from_numpy(coors_np).cuda()
    num = torch.tensor([n], dtype=torch.int32, device="cuda")
    r = pkg.subm_conv(feat, coors, num, p, w, keep_workspace=True)
    assert r["status"] == 0
    pairs, pnum = pkg.rulebook_export(p, 1, 0, r["workspace"], num)
    P_pairs = int(pnum.sum())
    ws, out = r["workspace"], r["features"]
    flush = torch.empty(160 << 20, dtype=torch.uint8, device="cuda")     # larger than L2: written between calls

    def step():
        flush.fill_(1)
        pkg.subm_conv_into(feat, coors, num, p, w, out, ws)

    def flush_only():
        flush.fill_(1)

    ms_both, clocks = _clocked(step, max(args.steps, 20), args.warmup)
    ms_flush, _ = _clocked(flush_only, max(args.steps, 20), args.warmup)
    ms = ms_both - ms_flush
    stages = pkg.profile(lambda: pkg.subm_conv_into(feat, coors, num, p, w, out, ws))
    flops = 2.0 * P_pairs * 16 * 16
    byts = n * 16 * 4 * 2 + 27 * 16 * 16 * 4 + 16.0 * n
    pk = peaks()
    ach = byts / (ms / 1e3) / 1e9
    sys.path.insert(0, ROOT)
    from oracle import binding as oracle
    t0 = time.perf_counter()
    reps = 5
    for _ in range(reps):
        op, on_, st = oracle.subm_rulebook(coors_np, n, layer.out_shape, maxV)
        oracle.conv_apply(feat_np, op, on_, W, n)
    cpu_s = (time.perf_counter() - t0) / reps
    w.close()
    return dict(metric="microseconds per SubMConv3d 16->16 call (rulebook + contraction, fp32, batch 1)", value=ms * 1e3,
                unit="us", n_gpus=1, steps=max(args.steps, 20), warmup=max(args.warmup, 3), ms_per_step=ms,
                higher_is_better=False, scaling="weak", vs_baseline=None, dtype="f32", data="synthetic",
                config=dict(workload="subm16", description=wl["desc"], active_voxels=n, pairs=P_pairs,
                            l2="160 MB written between calls (its time, measured alone, is subtracted)"),
                gpu_launches=len(stages) * max(args.steps, 20), clocks=clocks,
                kernels={name: round(t, 4) for name, t in stages},
                roofline=dict(bound="hbm", achieved=ach, peak=pk["hbm"], unit="GB/s", frac=ach / pk["hbm"], traffic=None,
                              kernel="whole call (5 launches)", tflops=flops / (ms / 1e3) / 1e12, peak_source=pk["source"]),
                cpu_baseline=dict(value=cpu_s * 1e6, unit="us", cores=1, kind="port",
                                  sample=f"mean of {reps} oracle calls (rulebook + contraction), one host thread"))


def detect_latency(pkg, frames_n=24, warm=6):
    """Frame -> kept boxes at batch 1 on 20,000-point frames (the reference's end-to-end configuration, random-init
    weights): host points in pinned memory, H2D, front end, fp16 neck + head (torch convolutions), fused decode +
    score filter, rotated NMS, D2H of the kept boxes, then a synchronisation, as in the reference's loop body."""
    import torch

    wl = WORKLOADS["single"]
    frames, sizes = make_frames(pkg, wl, frames_n, 0)
    P = wl["points"]
    w, sc, sh = pkg.random_weights()
    bb = pkg.Backbone(wl["max_voxels"], w, sc, sh, dtype=pkg.F16)
    blobs = pkg.detector.random_neck_weights()
    det = pkg.detector.Detector(bb, pkg.detector.Neck2D(blobs))
    h_pts = torch.from_numpy(frames).pin_memory()
    h_sizes = torch.from_numpy(sizes).pin_memory()
    d_pts = torch.empty((1, P, 4), device="cuda")
    d_sizes = torch.empty((1,), dtype=torch.int32, device="cuda")
    d_pts.copy_(h_pts[:1])
    d_sizes.copy_(h_sizes[:1])
    # a classification bias that lets a few hundred anchors through, as a trained head would
    logits = det(d_pts, d_sizes)["heads"]["cls"][0, :, 0].float().cpu().numpy()
    thr = float(np.log(pkg.schedule.SCORE_THRESHOLD / (1 - pkg.schedule.SCORE_THRESHOLD)))
    blobs["bbox_head.tasks.0.conv_cls.bias"] = blobs["bbox_head.tasks.0.conv_cls.bias"] + np.float32(thr - np.sort(logits)[-300])
    det = pkg.detector.Detector(bb, pkg.detector.Neck2D(blobs))
    ws = torch.empty(bb.workspace_bytes(1, P), dtype=torch.uint8, device="cuda")
    bev = torch.empty(bb.dense_shape(1), dtype=torch.float16, device="cuda")
    h_boxes = torch.empty((1, pkg.schedule.MAX_BOX_NUM, 9)).pin_memory()
    h_num = torch.empty((1,), dtype=torch.int32).pin_memory()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
    stage_ms, wall, kept = np.zeros(4), [], []
    for f in range(warm + frames_n):
        i = f % frames_n
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        ev[0].record()
        d_pts.copy_(h_pts[i:i + 1], non_blocking=True)
        d_sizes.copy_(h_sizes[i:i + 1], non_blocking=True)
        ev[1].record()
        bb.run(d_pts, d_sizes, ws, bev)
        ev[2].record()
        heads = det.neck(bev)
        ev[3].record()
        flt = pkg.filter_boxes(heads["box"], heads["cls"], heads["iou"], heads["dir"], det.filter, anchors=det.anchors)
        boxes, num = pkg.rotated_nms(flt["box"], flt["valid"], det.nms_thresh)
        h_boxes.copy_(boxes, non_blocking=True)
        h_num.copy_(num, non_blocking=True)
        ev[4].record()
        torch.cuda.synchronize()
        if f >= warm:
            wall.append((time.perf_counter() - t0) * 1e3)
            stage_ms += [ev[j].elapsed_time(ev[j + 1]) for j in range(4)]
            kept.append(int(h_num[0]))
    # the same chain recorded once into a CUDA graph: H2D into its input buffers, one graph launch, D2H
    det.capture(P)
    gwall = []
    for f in range(warm + frames_n):
        i = f % frames_n
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = det.replay(h_pts[i:i + 1], h_sizes[i:i + 1], read_back_status=False)
        h_boxes.copy_(out["boxes"], non_blocking=True)
        h_num.copy_(out["num"], non_blocking=True)
        torch.cuda.synchronize()
        if f >= warm:
            gwall.append((time.perf_counter() - t0) * 1e3)
    bb.close()
    stage_ms /= frames_n
    return dict(workload="20,000-point frames, batch 1, random-init weights", frames=frames_n,
                graph_latency_ms_median=float(np.median(gwall)), graph_latency_ms_mean=float(np.mean(gwall)),
                latency_ms_median=float(np.median(wall)), latency_ms_mean=float(np.mean(wall)),
                device_ms=dict(h2d=round(float(stage_ms[0]), 4), front_end=round(float(stage_ms[1]), 4),
                               neck_head_torch=round(float(stage_ms[2]), 4), filter_nms_d2h=round(float(stage_ms[3]), 4)),
                kept_boxes_mean=float(np.mean(kept)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="sweep", choices=sorted(WORKLOADS))
    ap.add_argument("--frames", type=int, default=0, help="frames per GPU per step (default: the workload's)")
    ap.add_argument("--batch", type=int, default=0, help="frames per launch group")
    ap.add_argument("--streams", type=int, default=0, help="launch groups in flight per GPU (default: the workload's, else 4)")
    ap.add_argument("--graphs", action="store_true", help="replay each launch group from a CUDA graph")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--detect", action="store_true", help="(kept for compatibility: the 1-GPU line always carries `detect`)")
    ap.add_argument("--no-detect", action="store_true", help="leave the frame -> boxes latency object out")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)

    if args.gpus > 1 and "RANK" not in os.environ:
        # started by hand without torchrun: start one rank per GPU of this node the way the launcher would
        port = str(29500 + os.getpid() % 1000)
        os.execv(sys.executable, [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                                  f"--nproc-per-node={args.gpus}", "--master-addr", "127.0.0.1", "--master-port", port,
                                  os.path.abspath(__file__), *sys.argv[1:]])
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    pkg = load_package()
    wl = dict(WORKLOADS[args.workload])
    if args.frames:
        wl["frames"] = args.frames
    if args.batch:
        wl["batch"] = args.batch
    if not args.streams:
        args.streams = wl.get("streams", 4)

    if args.impl == "reference":
        run_reference(args, pkg, wl, rank, world)
        return

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # NCCL announces its version on stdout when the communicator comes up: that happens here, with stdout
        # pointed at stderr, so that the benchmark's own stdout carries nothing but its JSON line
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)
    pkg.lib()

    if args.workload in ("voxelize", "subm16"):
        # the two small cases are single-GPU measurements with loops of their own
        if rank == 0:
            line = run_voxelize(args, pkg, wl) if args.workload == "voxelize" else run_subm16(args, pkg, wl)
            print(json.dumps(line), flush=True)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    F, P, B = wl["frames"], wl["points"], wl["batch"]
    frames, sizes = make_frames(pkg, wl, F, pkg.sharding.first_frame(rank, F))
    h_pts = torch.from_numpy(frames).pin_memory()
    h_sizes = torch.from_numpy(sizes).pin_memory()
    h_num = torch.zeros(F, dtype=torch.int32).pin_memory()
    h_status = torch.zeros(F, dtype=torch.int32).pin_memory()
    d_pts = h_pts.cuda()
    d_sizes = h_sizes.cuda()

    w, sc, sh = pkg.random_weights()
    bb = pkg.Backbone(wl["max_voxels"], w, sc, sh, dtype=pkg.F16)
    pipe = pkg.Pipeline(bb, B, P, nstreams=args.streams)
    if args.graphs:
        pipe.use_graphs(True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    sampler.start()
    for i in range(max(args.warmup, 3)):
        pipe.run_device(d_pts, d_sizes)
        if i == 0:   # fail fast if a kernel reported a bounded-wait timeout or a capacity problem
            bad = pipe.status_bits()
            if bad & ~pkg.STATUS_VOXEL_OVERFLOW:
                sampler.stop()
                raise SystemExit(f"device status {bad:#x} after the first pass: aborting the benchmark")
    barrier()
    launches0 = pkg.launch_count()
    t0 = time.perf_counter()
    dev_ms = 0.0
    for _ in range(args.steps):
        dev_ms += pipe.run_device(d_pts, d_sizes)      # CUDA events on the pipeline's own streams
    barrier()
    wall_ms = (time.perf_counter() - t0) * 1e3
    launches = pkg.launch_count() - launches0
    clocks = sampler.stop(t0, time.perf_counter())
    # a pipeline's status words collect every group of a run: this is the status of the last timed step
    status_bits = pipe.status_bits()

    # end to end through the host-buffer entry point: H2D of the points and D2H of counts + status inside
    for _ in range(2):
        pipe.run_host(h_pts, h_sizes, h_num, h_status)
    barrier()
    e2e_ms = 0.0
    for _ in range(args.steps):
        e2e_ms += pipe.run_host(h_pts, h_sizes, h_num, h_status)
    barrier()
    status_bits |= int(np.bitwise_or.reduce(h_status.numpy())) | pipe.status_bits()
    # the same with every group's BEV maps copied to pinned host memory as well (9 MB per frame)
    h_dense = torch.empty((args.streams,) + tuple(bb.dense_shape(B)), dtype=torch.float16).pin_memory()
    pipe.run_host_bev(h_pts, h_sizes, h_num, h_status, h_dense)
    barrier()
    bev_ms = 0.0
    for _ in range(args.steps):
        bev_ms += pipe.run_host_bev(h_pts, h_sizes, h_num, h_status, h_dense)
    barrier()
    status_bits |= pipe.status_bits()
    dense_bytes_per_frame = int(np.prod(bb.dense_shape(1))) * 2

    t = torch.tensor([dev_ms, e2e_ms, wall_ms, bev_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        # OR over ranks, bit by bit (a condition on any rank must reach the printed line)
        bits = torch.tensor([(status_bits >> i) & 1 for i in range(16)], dtype=torch.int64, device="cuda")
        dist.all_reduce(bits, op=dist.ReduceOp.MAX)
        status_bits = sum(int(v) << i for i, v in enumerate(bits.cpu()))
    dev_ms, e2e_ms, wall_ms, bev_ms = [float(v) for v in t.cpu()]
    total_frames = F * args.steps * world
    value = total_frames / (dev_ms / 1e3)
    e2e = total_frames / (e2e_ms / 1e3)
    e2e_bev = total_frames / (bev_ms / 1e3)

    line = None
    if rank == 0:
        # per-kernel device times of one launch group, measured with events around every launch
        grp_pts, grp_sizes = d_pts[:B].contiguous(), d_sizes[:B].contiguous()
        ws = torch.empty(bb.workspace_bytes(B, P), dtype=torch.uint8, device="cuda")
        dense = torch.empty(bb.dense_shape(B), dtype=torch.float16, device="cuda")
        bb.run(grp_pts, grp_sizes, ws, dense)
        torch.cuda.synchronize()
        stages = pkg.profile(lambda: bb.run(grp_pts, grp_sizes, ws, dense))
        per_kernel = {}
        for name, ms in stages:
            k = per_kernel.setdefault(name.strip("()"), [0, 0.0])
            k[0] += 1
            k[1] += ms
        group_ms = sum(v[1] for v in per_kernel.values())
        # algorithmic work of that group: rows per layer from the device, pairs from the neighbour maps
        rows_in, rows_out, pairs = [], [], pkg.pair_counts(bb, grp_pts, grp_sizes, ws, dense)
        prev = int(bb.layer_view(ws, B, P, -1)[2].sum())
        for i in range(len(bb.layers)):
            n = int(bb.layer_view(ws, B, P, i)[2].sum())
            rows_in.append(prev)
            rows_out.append(n)
            prev = n
        costs = layer_costs(pkg, rows_in, rows_out, pairs)
        pk = peaks()
        is_conv = lambda n: n.startswith("conv_simt") or n.startswith("conv_umma")  # noqa: E731
        top = max(per_kernel, key=lambda n: per_kernel[n][1])
        # every conv kernel instance is attributed the layers it ran (same order as the schedule)
        conv_launch_order = [n.strip("()") for n, _ in stages if is_conv(n)]
        conv_ms = [ms for n, ms in stages if is_conv(n)]
        if is_conv(top):
            idx = [i for i, n in enumerate(conv_launch_order) if n == top]
            flops = sum(costs[i]["flops"] for i in idx)
            byts = sum(costs[i]["bytes"] for i in idx)
            ms = sum(conv_ms[i] for i in idx)
            tens = any(pkg.schedule.LAYERS[i].cin >= 32 for i in idx)
            if tens:
                # the launches are timed one by one, alone on the GPU: the burst figure is their denominator
                ach = flops / (ms / 1e3) / 1e12
                roof = dict(bound="tensor", achieved=ach, peak=pk["tensor"], unit="TFLOP/s",
                            frac=ach / pk["tensor"], traffic=None, peak_kind="burst (kernel timed alone)")
            else:
                ach = byts / (ms / 1e3) / 1e9
                roof = dict(bound="hbm", achieved=ach, peak=pk["hbm"], unit="GB/s", frac=ach / pk["hbm"], traffic=None)
            per_frame, traffic_src = measured_traffic(args.workload, top)
            roof.update(kernel=top, launches=len(idx), avg_launch_ms=ms / len(idx), peak_source=pk["source"],
                        algorithmic_bytes=byts / len(idx), traffic=per_frame * B if per_frame else None,
                        traffic_source=traffic_src)
            l2sm = measured_l2_to_sm(args.workload, top)
            if l2sm:
                roof["l2_to_sm_bytes_quarter_resolution_launch"] = l2sm * B
        else:
            vox_rows = int(bb.layer_view(ws, B, P, -1)[2].sum())
            byts = 16.0 * float(grp_sizes.sum()) + vox_rows * (16 + 8 + 4) + 4 * B
            ms = per_kernel[top][1]
            ach = byts / (ms / 1e3) / 1e9
            roof = dict(bound="hbm", achieved=ach, peak=pk["hbm"], unit="GB/s", frac=ach / pk["hbm"], traffic=None,
                        kernel=top, launches=per_kernel[top][0], avg_launch_ms=ms / per_kernel[top][0],
                        peak_source=pk["source"])
        total_flops = sum(c["flops"] for c in costs)
        total_bytes = sum(c["bytes"] for c in costs)
        # the whole job against the sustained peaks: pair flops and algorithmic bytes of one frame x frames per second
        whole = dict(pair_tflops=total_flops / B * value / world / 1e12,
                     frac_of_sustained_tensor_peak=total_flops / B * value / world / 1e12 / pk["tensor_sustained"],
                     algorithmic_gbps=total_bytes / B * value / world / 1e9,
                     frac_of_hbm_peak=total_bytes / B * value / world / 1e9 / pk["hbm"], per="GPU")
        line = dict(metric=METRIC, value=value, unit="frames/s", n_gpus=world, steps=args.steps,
                    warmup=max(args.warmup, 3), ms_per_step=dev_ms / args.steps, higher_is_better=True,
                    scaling="weak", vs_baseline=None, dtype="f16", data="synthetic",
                    config=dict(workload=args.workload, description=wl["desc"], points_per_frame=P,
                                frames_per_gpu_per_step=F, frames_per_launch_group=B, streams=args.streams, cuda_graphs=bool(args.graphs),
                                max_voxels=wl["max_voxels"], layers=len(bb.layers),
                                l2="inputs larger than L2 (points of one step: %.0f MB)" % (F * P * 16 / 1e6),
                                parallelism=f"frames sharded over {world} GPU(s), no collective"),
                    e2e=dict(value=e2e, unit="frames/s", h2d_bytes_per_step=F * P * 16 + F * 4,
                             d2h_bytes_per_step=F * 4 + (F + B - 1) // B * 4,
                             result="final row counts and status words; the dense BEV map stays on the device for the "
                                    "2D head, as in the reference, which copies only boxes back"),
                    e2e_with_bev=dict(value=e2e_bev, unit="frames/s", h2d_bytes_per_step=F * P * 16 + F * 4,
                                      d2h_bytes_per_step=F * 4 + (F + B - 1) // B * 4 + F * dense_bytes_per_frame,
                                      result="the same plus every frame's dense BEV map copied to pinned host memory"),
                    gpu_launches=int(launches), clocks=clocks, roofline=roof, whole_job=whole,
                    wall_ms_per_step=wall_ms / args.steps, status_bits=status_bits,
                    group_profile=dict(frames=B, total_ms=group_ms,
                                       gflop_per_frame=total_flops / B / 1e9,
                                       kernels={n: dict(launches=v[0], ms=round(v[1], 4)) for n, v in
                                                sorted(per_kernel.items(), key=lambda kv: -kv[1][1])},
                                       # per conv layer: launch time, algorithmic GB/s and TFLOP/s (pair flops)
                                       layers=[dict(name=c["name"], kernel=k, ms=round(ms, 4),
                                                    gbps=round(c["bytes"] / (ms / 1e3) / 1e9, 1),
                                                    tflops=round(c["flops"] / (ms / 1e3) / 1e12, 2))
                                               for c, k, ms in zip(costs, conv_launch_order, conv_ms)]))
        if world == 1 and not args.no_cpu_baseline:
            info, _, _ = cpu_baseline(pkg, wl, frames, sizes)
            line["cpu_baseline"] = info
        else:
            line["cpu_baseline"] = None
    pipe.close()
    bb.close()
    if rank == 0 and world == 1 and not args.no_detect:
        try:   # frame -> boxes at batch 1 (the end-to-end configuration), in the record of every 1-GPU run
            line["detect"] = detect_latency(pkg)
        except Exception as exc:   # the 2D neck needs torch's convolutions; the headline does not depend on it
            line["detect"] = dict(error=f"{type(exc).__name__}: {exc}")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
