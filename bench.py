#!/usr/bin/env python
"""Benchmark of the sparse-convolution hot path: MinkUNet-34 inference forward
(fp16, random-init weights) over batches of synthetic indoor rooms.

    python bench.py --gpus N --steps K --warmup W          # this library
    python bench.py --impl reference --steps K --warmup W  # the reference's CPU path

Besides the headline (MinkUNet-34 voxels/s) the line carries, measured outside the timed
regions: ``kmap`` (kernel-map build alone over 4 x 250 000-voxel rooms, both generators:
Mcoords/s, algorithmic GB/s and fraction of the HBM copy bandwidth per stage), ``layers`` (single
layers on a 500 000-voxel room: 3x3x3 / stride-2 down / transposed up, widths 32..256, fp16 and
bf16), ``strong`` (the SAME 8-room batch divided among the ranks) and, with two or more ranks,
``config5`` (one 8 M-voxel LiDAR scene split by Morton range with a halo exchange).

One step = one pass of the whole path over one batch held by a rank: Morton
ordering of the voxels, coordinate hashing, kernel-map generation for every
resolution level, the 46 3x3x3 / 4 down / 4 up / 1x1x1 convolutions with their
fused BatchNorm/ReLU/residual epilogues, un-permutation of the logits.  Every
step sees a fresh ``Voxels`` object, so nothing (maps, orderings) is carried
over between steps.  ``value`` times the step with the batch already in HBM;
``e2e`` times the same step from pinned host buffers, with the host-to-device
copy of coordinates and features and the device-to-host copy of the logits
inside the timed region (on copy streams, overlapping the neighbouring step).

Ranks hold independent scene groups (no data-path collective): weak scaling.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "sparse-conv voxels/sec (MinkUNet fwd)"
UNIT = "voxels/s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--scenes", type=int, default=8, help="rooms per rank")
    ap.add_argument("--voxels", type=int, default=150000, help="voxels per room")
    ap.add_argument("--voxel-size", type=float, default=0.02)
    ap.add_argument("--mode", choices=["raster_crop", "sample"], default="raster_crop")
    ap.add_argument("--cpu-sample-voxels", type=int, default=150000)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--layers", action="store_true", help="print a per-launch table of the convolutions to stderr")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the kernel-map, single-layer, strong-scaling and partitioned-scene measurements")
    ap.add_argument("--lidar-voxels", type=int, default=8000000, help="size of the partitioned scene (2+ ranks)")
    return ap.parse_args()


# --------------------------------------------------------------------------- workload


def make_batch(args, rank, scene_ids=None):
    """Rooms ``scene_ids`` (default: the rank's own group of ``--scenes`` rooms) as one batch."""
    from warpconvnet_b200.datasets import synthetic
    if scene_ids is None:
        scene_ids = [rank * args.scenes + s for s in range(args.scenes)]
    scenes = [synthetic.room_scene(args.voxels, args.voxel_size, 200 + s, args.mode) for s in scene_ids]
    coords, offsets = synthetic.batch_scenes(scenes)
    feats = np.random.default_rng(1000 + scene_ids[0]).random((len(coords), 3), dtype=np.float32)
    return coords, offsets, feats


def make_model():
    from warpconvnet_b200.examples.mink_unet import MinkUNet34, randomize_batchnorm_
    torch.manual_seed(0)
    model = MinkUNet34(3, 20)
    randomize_batchnorm_(model, 1)
    return model.eval()


# --------------------------------------------------------------------------- clocks


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples of one GPU while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def mark(self):
        """Index of the next sample; samples between two marks belong to a timed region."""
        return len(self.lines)

    def stop(self, first=0, last=None):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        window = self.lines[first:last] if last is not None and last > first else self.lines[first:]
        for ln in window:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                smax = float(parts[1])
            except ValueError:
                continue
            for nm, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm)}


# --------------------------------------------------------------------------- CPU arm (the reference's own path restated)


def cpu_forward_timed(args, repeats):
    """The reference's CPU-runnable path — explicit-GEMM convolutions on torch CPU
    tensors + the kernel-map restatement — over one room; returns (voxels/s, info)."""
    from oracle import sparse_conv as osc
    from warpconvnet_b200.datasets import synthetic
    torch.set_num_threads(os.cpu_count() or 1)
    model = make_model()
    sd = model.state_dict()
    n = args.cpu_sample_voxels
    xyz = synthetic.room_scene(n, args.voxel_size, 200, args.mode)
    coords = np.concatenate([np.zeros((len(xyz), 1), np.int32), xyz], 1)
    feats = torch.rand(n, 3, generator=torch.Generator().manual_seed(0))
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        osc.minkunet_forward(sd, coords, feats)
        times.append(time.perf_counter() - t0)
    return n, times


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n, _ = cpu_forward_timed(args, max(args.warmup, 1))
    n, times = cpu_forward_timed(args, args.steps)
    total = sum(times)
    value = n * len(times) / total
    cores = torch.get_num_threads()
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "impl": "reference",
        "config": workload_config(args, note="CPU arm: each step is one room of the workload"),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"one {args.mode} room of {n} voxels per step, fp32, MinkUNet-34 forward"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(args, note=None):
    cfg = {"workload": f"MinkUNet-34 inference forward, fp16, batch of {args.scenes} synthetic rooms x "
                       f"{args.voxels} voxels at {args.voxel_size} m ({args.mode}), 3 input channels, 20 classes; "
                       "one scene group per GPU, no communication",
           "scenes_per_gpu": args.scenes, "voxels_per_scene": args.voxels, "generator": args.mode,
           "l2": "flushed between steps (256 MiB write); per-step working set is also far larger than L2",
           "pipelining": "two steps in flight on alternating CUDA streams (a step's coordinate front overlaps the "
                         "previous step's convolutions); every step does all of its work inside the timed region",
           "step": "morton sort + hash/kernel maps (rebuilt every step) + all convolutions + unpermute"}
    if note:
        cfg["note"] = note
    return cfg


# --------------------------------------------------------------------------- GPU arm


class ConvProfile:
    """Per-launch durations and useful FLOPs of the convolution launches of a step.

    While a step runs, every fused-convolution call is recorded (its arguments stay alive).
    After the step the recorded launches are replayed in order behind a device-side delay, so
    the host is far ahead of the GPU and each launch is bracketed by CUDA events on the
    launching stream without host-induced gaps."""

    def __init__(self):
        self.calls = []    # (callable, nbr tensor or (pairs, M, K), c_in, c_out, kind) of the step being recorded
        self.records = []  # (ms, pairs, M, K, c_in, c_out, kind) of replayed launches
        self._pairs = {}

    def replay(self):
        torch.cuda.synchronize()
        torch.cuda._sleep(200_000_000)  # ~0.1 s: time for the host to enqueue every launch below
        evs = []
        for fn, nbr, c_in, c_out, kind in self.calls:
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            evs.append((s, e))
        torch.cuda.synchronize()
        for (s, e), (fn, nbr, c_in, c_out, kind) in zip(evs, self.calls):
            if isinstance(nbr, tuple):  # a layer run from the input side: one pair per output row
                pairs, M, K = nbr
                self.records.append((s.elapsed_time(e), pairs, M, K, c_in, c_out, kind))
                continue
            key = nbr.data_ptr()
            if key not in self._pairs:
                self._pairs[key] = int((nbr >= 0).sum().item())
            self.records.append((s.elapsed_time(e), self._pairs[key], nbr.shape[1], nbr.shape[0], c_in, c_out, kind))
        self.calls = []
        self._pairs = {}

    def summarise(self):
        out = {"launches": 0, "ms": 0.0, "flop": 0.0, "tc_launches": 0, "tc_ms": 0.0, "tc_flop": 0.0}
        for ms, pairs, M, K, c_in, c_out, kind in self.records:
            fl = 2.0 * pairs * c_in * c_out
            out["launches"] += 1; out["ms"] += ms; out["flop"] += fl
            if kind == "tcgen05":
                out["tc_launches"] += 1; out["tc_ms"] += ms; out["tc_flop"] += fl
        return out

    def by_shape(self, steps, peak_tf, peak_gbs, top=8):
        """The tensor-core launches of a step grouped by shape, slowest group first: launches and
        milliseconds per step, useful TFLOP/s, and the fraction of the roofline that binds the
        shape (max of FLOP time at the tensor peak and algorithmic-byte time at the HBM peak)."""
        groups = {}
        for ms, pairs, M, K, c_in, c_out, kind in self.records:
            if kind != "tcgen05":
                continue
            g = groups.setdefault((K, M, c_in, c_out), [0, 0.0, 0.0, 0.0])
            g[0] += 1
            g[1] += ms
            g[2] += 2.0 * pairs * c_in * c_out
            g[3] += 2.0 * (M * c_in + M * c_out + K * c_in * c_out) + 4.0 * K * M  # fp16 rows in/out + weights + table
        out = []
        for (K, M, c_in, c_out), (cnt, ms, fl, by) in sorted(groups.items(), key=lambda kv: -kv[1][1])[:top]:
            t_tc, t_hbm = fl / (peak_tf * 1e12), by / (peak_gbs * 1e9)
            out.append({"offsets": K, "rows": M, "c_in": c_in, "c_out": c_out, "launches_per_step": cnt / steps,
                        "ms_per_step": ms / steps, "useful_tflops": fl / ms / 1e9 if ms > 0 else 0.0,
                        "bound": "tensor" if t_tc > t_hbm else "hbm",
                        "roofline_frac": max(t_tc, t_hbm) / (ms * 1e-3) if ms > 0 else 0.0})
        return out

    def table(self, last_n):
        rows = []
        for ms, pairs, M, K, c_in, c_out, kind in self.records[-last_n:]:
            rows.append(f"{kind:8s} K={K:2d} M={M:8d} {c_in:4d}->{c_out:4d} pairs/M={pairs / max(M, 1):5.2f} "
                        f"{ms * 1e3:8.1f} us {2.0 * pairs * c_in * c_out / ms / 1e9:7.1f} TFLOP/s")
        return "\n".join(rows)


def install_conv_profiler(profile):
    """Wrap the fused-convolution entries (the functional one and the two launch records the network
    plan uses) so that each call of a step is recorded for replay."""
    import warpconvnet_b200.nn.functional.sparse_conv as F
    from warpconvnet_b200._native import query_bytes, dtype_code
    orig = F.sparse_conv_fused
    orig_launch = F.FusedConvLaunch.__call__
    orig_rows = F.FusedRowsLaunch.__call__

    def rows_launch(self, feats, dst_rows, num_out, residual=None, out=None):
        res = orig_rows(self, feats, dst_rows, num_out, residual, out)
        profile.calls.append((lambda: orig_rows(self, feats, dst_rows, num_out, residual, res),
                              (num_out, num_out, self.K), self.c_in, self.c_out, "tcgen05"))
        return res

    def wrapped(in_features, weight, kernel_map, num_out_coords, *rest, **kw):
        out = orig(in_features, weight, kernel_map, num_out_coords, *rest, **kw)
        K, c_in, c_out = weight.shape
        tc = in_features.dtype != torch.float32 and query_bytes(
            "wcn_conv_packed_weight_bytes", 0, K, c_in, c_out, dtype_code(in_features.dtype)) > 0
        profile.calls.append((lambda: orig(in_features, weight, kernel_map, num_out_coords, *rest, **kw),
                              kernel_map.neighbor_table(num_out_coords), c_in, c_out, "tcgen05" if tc else "simt"))
        return out

    def launch(self, feats, nbr, out_rows, num_out, residual=None, out=None):
        res = orig_launch(self, feats, nbr, out_rows, num_out, residual, out)
        profile.calls.append((lambda: orig_launch(self, feats, nbr, out_rows, num_out, residual, res),
                              nbr, self.c_in, self.c_out, "tcgen05" if self.packed is not None else "simt"))
        return res

    F.sparse_conv_fused = wrapped
    F.FusedConvLaunch.__call__ = launch
    F.FusedRowsLaunch.__call__ = rows_launch

    def restore():
        F.sparse_conv_fused = orig
        F.FusedConvLaunch.__call__ = orig_launch
        F.FusedRowsLaunch.__call__ = orig_rows
    return restore


# DRAM bytes (read + write) of one 3x3x3 C = 96 fp16 launch over 500 000 rows, from the ncu capture
# summarised under profiles/ (153 MB read + 63 MB written; the algorithmic bytes are 248 MB).
NCU_DRAM_BYTES_C96_500K = 216e6


def measure_strong(args, rank, world, dev, model, forward_of, timed, flush, weak_ms_per_step, weak_voxels, lanes, lane,
                   join_lanes):
    """Strong scaling of the batched workload: the SAME batch of ``--scenes`` rooms (1.2 M voxels)
    divided among the ranks in contiguous scene groups, no communication; a rank without rooms
    idles.  Reported as whole-job voxels/s with the slowest rank's time."""
    import torch.distributed as dist
    from warpconvnet_b200.dist.sharding import split_scene_groups
    total = args.scenes * args.voxels
    if world == 1:
        return {"n_gpus": 1, "voxels_total": weak_voxels, "ms_per_step": weak_ms_per_step,
                "value": weak_voxels / (weak_ms_per_step * 1e-3), "unit": UNIT, "scenes_per_rank": [args.scenes]}
    groups = split_scene_groups([i * args.voxels for i in range(args.scenes + 1)], world)
    first, last = groups[rank]
    step = None
    if last > first:
        coords_np, offsets_np, feats_np = make_batch(args, rank, scene_ids=list(range(first, last)))
        xyz = torch.from_numpy(np.ascontiguousarray(coords_np[:, 1:])).to(dev)
        feats = torch.from_numpy(feats_np).half().to(dev)
        fwd = forward_of(torch.from_numpy(offsets_np))

        def step():
            lane["i"] ^= 1
            with torch.cuda.stream(lanes[lane["i"]]):  # two steps in flight, as in the headline loop
                flush.zero_()
                return fwd(xyz, feats)
    run = step if step is not None else (lambda: None)
    steps = max(args.steps, 5)
    for _ in range(3):
        run()
    ms = timed(run, steps, finish=join_lanes)
    return {"n_gpus": world, "voxels_total": total, "ms_per_step": ms / steps, "value": total * steps / (ms * 1e-3),
            "unit": UNIT, "scenes_per_rank": [g[1] - g[0] for g in groups],
            "limit": "per-forward host work (one Python thread per rank) once a rank holds one room or less"}


def measure_config5(args, rank, world, dev):
    """One large LiDAR scene split by Morton range over the ranks: one 3x3x3 stride-1 bf16 convolution,
    C = 128, with the one-voxel halo exchange; plus a 300 000-voxel scene on which the ranks' rows are
    compared bit for bit with the single-GPU convolution."""
    from warpconvnet_b200.examples import partitioned_conv_bench as pcb
    coords, info = pcb.shared_scene(args.lidar_voxels, 4, 8192, dev, rank, world)
    res = pcb.measure(coords, 128, torch.bfloat16, 10, rank, world)
    del coords
    small, _ = pcb.shared_scene(300000, 4, 2048, dev, rank, world)
    chk = pcb.measure(small, 128, torch.bfloat16, 2, rank, world, check=True)
    res["scene"] = info
    res["check_scene_voxels"] = chk["voxels"]
    res["max_abs_diff_vs_single_gpu"] = chk.get("max_abs_diff_vs_single_gpu")
    return res


def run_gpu_arm(args):
    import torch.distributed as dist
    from warpconvnet_b200 import POINT_ORDERING, Voxels
    from warpconvnet_b200 import _native

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        # NCCL announces its version on stdout when the first communicator comes up; stdout
        # carries exactly one JSON line, so that announcement is sent to stderr.
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=dev)
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)
    _native.lib()  # fail loudly now if the library is missing

    coords_np, offsets_np, feats_np = make_batch(args, rank)
    n_vox = len(coords_np)
    model = make_model().to(dev).half()
    xyz_host = torch.from_numpy(np.ascontiguousarray(coords_np[:, 1:])).pin_memory()
    feats_host = torch.from_numpy(feats_np).half().pin_memory()
    offsets = torch.from_numpy(offsets_np)
    logits_host = torch.empty((n_vox, 20), dtype=torch.float16).pin_memory()
    xyz_dev, feats_dev = xyz_host.to(dev), feats_host.to(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def make_forward(batch_offsets):
        def fwd(xyz, feats):
            vox = Voxels(xyz, feats, offsets=batch_offsets)
            ordered = vox.sort(POINT_ORDERING.MORTON_XYZ)
            return model(ordered, restore_order=True)  # logits in the caller's row order
        return fwd

    forward = make_forward(offsets)

    # Consecutive steps are independent, so two are kept in flight on alternating streams: the front
    # of a step (Morton sort, coordinate pyramid with its four size read-backs) synchronises the host
    # with ITS stream only and runs while the other stream still executes the previous step's
    # convolutions.  Every tensor of a step is allocated, used and freed on the step's own stream.
    lanes = [torch.cuda.Stream(dev), torch.cuda.Stream(dev)]
    lane = {"i": 0}

    def step_resident():
        lane["i"] ^= 1
        with torch.cuda.stream(lanes[lane["i"]]):
            flush.zero_()
            return forward(xyz_dev, feats_dev)

    def join_lanes():
        cur = torch.cuda.current_stream(dev)
        for s in lanes:
            cur.wait_stream(s)

    # End-to-end step: the host->device copy of step i+1 and the device->host copy of step i run
    # on their own streams and overlap the compute of the neighbouring step (double-buffered
    # device inputs and pinned host outputs); every step still moves all of its bytes inside
    # the timed region.
    h2d, d2h = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    in_buf = [(torch.empty_like(xyz_dev), torch.empty_like(feats_dev)) for _ in range(2)]
    out_host = [logits_host, torch.empty_like(logits_host).pin_memory()]
    e2e = {"i": 0, "in_ready": [None, None], "done": [None, None], "out_copied": [None, None]}

    def prefetch(i):
        b = i % 2
        with torch.cuda.stream(h2d):
            if e2e["done"][b] is not None:
                h2d.wait_event(e2e["done"][b])  # the step that last read this buffer has finished
            in_buf[b][0].copy_(xyz_host, non_blocking=True)
            in_buf[b][1].copy_(feats_host, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(h2d)
            e2e["in_ready"][b] = ev

    def step_e2e():
        i = e2e["i"]
        b = i % 2  # input buffer b, output buffer b and stream b belong together
        if e2e["in_ready"][b] is None:
            prefetch(i)
        main = lanes[b]
        with torch.cuda.stream(main):
            main.wait_event(e2e["in_ready"][b])
            e2e["in_ready"][b] = None
            prefetch(i + 1)  # overlaps this step's compute
            flush.zero_()
            logits = forward(in_buf[b][0], in_buf[b][1])
            done = torch.cuda.Event()
            done.record(main)
            e2e["done"][b] = done
            logits.record_stream(d2h)
            with torch.cuda.stream(d2h):
                d2h.wait_event(done)
                out_host[b].copy_(logits, non_blocking=True)  # overlaps the next step's compute
        e2e["i"] = i + 1

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, finish=None):
        barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for ln in lanes:
            ln.wait_event(s)  # nothing of the timed steps starts before the start event
        for _ in range(steps):
            fn()
        if finish is not None:
            finish()  # work on other streams that belongs to the timed steps
        e.record()
        barrier()
        ms = torch.tensor([s.elapsed_time(e)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    sampler = ClockSampler(local_rank)
    sampler.start()  # nvidia-smi needs about a second before its first sample
    with torch.no_grad():
        for _ in range(max(args.warmup, 3)):
            step_resident()
        _native.check_device_status(dev)
        mark0 = sampler.mark()
        before = _native.launches_total()
        ms = timed(step_resident, args.steps, finish=join_lanes)
        launches = _native.launches_total() - before
        for _ in range(2):
            step_e2e()
        # the last step's device-to-host copy runs on the copy stream: the end event follows it
        def join_e2e():
            join_lanes()
            torch.cuda.current_stream(dev).wait_stream(d2h)

        ms_e2e = timed(step_e2e, args.steps, finish=join_e2e)
        mark1 = sampler.mark()
        _native.check_device_status(dev)
        time.sleep(0.06)
        clocks = sampler.stop(mark0, max(mark1, mark0 + 1))
        clocks["window"] = "device-resident and end-to-end timed regions"

        # roofline of the dominant kernel: per-launch CUDA events over a timed region of its own
        prof_steps = min(args.steps, 3)
        for attempt in range(2):
            profile = ConvProfile()
            restore = install_conv_profiler(profile)
            barrier()
            for _ in range(prof_steps):
                step_resident()
                profile.replay()
            barrier()
            restore()
            _native.check_device_status(dev)  # a kernel that gave up would make every later launch a no-op
            prof = profile.summarise()
            # sanity: the convolutions cannot take less than a third of a step nor exceed the tensor peak;
            # a reading outside that is a measurement glitch and is taken again once
            share = (prof["ms"] / prof_steps) / (ms / args.steps)
            if 0.3 < share < 1.2:
                break
        profile_retaken = attempt
        if args.layers and rank == 0:
            print(profile.table(len(profile.records) // prof_steps), file=sys.stderr)

        # ---- further measurements, each outside the two timed regions above
        strong = config5 = kmap = layers = None
        if not args.no_extras:
            strong = measure_strong(args, rank, world, dev, model, forward_of=make_forward, timed=timed, flush=flush,
                                    weak_ms_per_step=ms / args.steps, weak_voxels=n_vox, lanes=lanes, lane=lane,
                                    join_lanes=join_lanes)
            if world > 1:
                config5 = measure_config5(args, rank, world, dev)
            if rank == 0:
                from warpconvnet_b200.examples import kernel_map_bench, layer_sweep
                kmap = []
                for mode in ("raster_crop", "sample"):  # rows as generated (voxel table), then Morton-ordered (bricks)
                    kmap += kernel_map_bench.measure(4, 250000, 0.02, mode, iters=6, dev=dev, flush=flush)
                    kmap += kernel_map_bench.measure(4, 250000, 0.02, mode, iters=6, sort=True, dev=dev, flush=flush)
                layers = layer_sweep.measure(500000, 0.01, "raster_crop", iters=5, dev=dev, flush=flush)
            _native.check_device_status(dev)
            barrier()

    total_vox = n_vox * world  # every rank holds a batch of the same size
    if world > 1:
        t = torch.tensor([n_vox], device=dev, dtype=torch.int64)
        dist.all_reduce(t)
        total_vox = int(t.item())
    value = total_vox * args.steps / (ms * 1e-3)
    e2e_value = total_vox * args.steps / (ms_e2e * 1e-3)

    if rank == 0:
        peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
        if os.path.isfile(peaks_path):
            peaks = json.load(open(peaks_path))
            peak_tf, peak_src = float(peaks["bf16_tflops_sustained"]), "measured sustained bf16 (MEASURED_PEAKS.json)"
            peak_gbs = float(peaks["hbm_gbs"])
        else:
            peak_tf, peak_src, peak_gbs = 1400.0, "fallback sustained figure", 6650.0
        achieved_tf = prof["tc_flop"] / (prof["tc_ms"] * 1e-3) / 1e12 if prof["tc_ms"] > 0 else 0.0
        shapes = profile.by_shape(prof_steps, peak_tf, peak_gbs)
        dominant = shapes[0] if shapes else None
        roofline = {
            "bound": "tensor", "achieved": achieved_tf, "peak": peak_tf, "unit": "TFLOP/s",
            "frac": achieved_tf / peak_tf,
            # DRAM bytes per launch of the dominant shape (3x3x3, C = 96, the finest level): ncu's
            # dram__bytes_read + dram__bytes_write on a 500 000-row launch of the same shape
            # (profiles/), scaled to this launch's rows; traffic grows in proportion to the rows.
            "traffic": (NCU_DRAM_BYTES_C96_500K * dominant["rows"] / 500000.0
                        if dominant and (dominant["c_in"], dominant["c_out"], dominant["offsets"]) == (96, 96, 27) else None),
            "traffic_of": "dominant shape, per launch", "peak_source": peak_src,
            "kernel": "conv_tcgen05_kernel + conv_rows_tcgen05_kernel (all tensor-core convolution launches of a step)",
            "useful_flop_per_step": prof["tc_flop"] / prof_steps, "launches_per_step": prof["tc_launches"] / prof_steps,
            "avg_launch_ms": prof["tc_ms"] / max(prof["tc_launches"], 1),
            "conv_share_of_step": (prof["ms"] / prof_steps) / (ms / args.steps),
            "profile_retaken": profile_retaken, "by_shape": shapes,
        }
        cpu = None
        if not args.no_cpu_baseline:
            n, _ = cpu_forward_timed(args, 1)
            n, times = cpu_forward_timed(args, 3)
            cpu = {"value": n * len(times) / sum(times), "unit": UNIT, "cores": torch.get_num_threads(),
                   "kind": "port", "sample": f"3 forwards of one {args.mode} room of {n} voxels, fp32, all host threads"}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": workload_config(args),
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": int(xyz_host.numel() * 4 + feats_host.numel() * 2),
                    "d2h_bytes_per_step": int(logits_host.numel() * 2)},
            "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu,
            "voxels_per_gpu": n_vox, "strong": strong, "kmap": kmap, "layers": layers, "config5": config5,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
