"""One large outdoor scene split across GPUs by Morton-code range: a 3x3x3 stride-1
convolution with a one-voxel NCCL halo exchange before it.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m warpconvnet_b200.examples.partitioned_conv_bench --voxels 8000000 --channels 128 --dtype bf16

Every rank builds the same seeded synthetic LiDAR scene, sorts it by Morton code, owns an
equal-count range, plans its halo once, then times (halo exchange + convolution) with CUDA
events; the slowest rank counts.  Rank 0 prints one JSON line; with --check it also runs
the whole scene on its own GPU and compares the owned rows of every rank bit for bit.
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np
import torch
import torch.distributed as dist

from .. import generate_kernel_map
from .._native import check_device_status
from ..datasets import synthetic
from ..dist.halo import morton_partition, partitioned_conv, plan_halo
from ..nn.functional.sparse_conv import sparse_conv_fused

DT = {"fp16": torch.float16, "bf16": torch.bfloat16}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--voxels", type=int, default=8000000)
    ap.add_argument("--sweeps", type=int, default=4)
    ap.add_argument("--azimuth-steps", type=int, default=8192)
    ap.add_argument("--channels", type=int, default=128)
    ap.add_argument("--dtype", default="bf16", choices=list(DT))
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--check", action="store_true")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    xyz, info = synthetic.lidar_scene(args.voxels, args.sweeps, args.azimuth_steps, seed=500)
    n = len(xyz)
    coords = torch.from_numpy(np.concatenate([np.zeros((n, 1), np.int32), xyz], 1)).to(dev)
    perm, bounds = morton_partition(coords, world)
    gc = coords[perm].contiguous()
    plan = plan_halo(gc, bounds, rank, world)
    lo, hi = bounds[rank], bounds[rank + 1]
    c, dt = args.channels, DT[args.dtype]
    g = torch.Generator(device="cpu").manual_seed(1)
    w = ((torch.rand(27, c, c, generator=g) * 2 - 1) * (3.0 / (27 * c)) ** 0.5 * 1.73).to(dev, dt)
    # features are a function of the global row, so every rank can make its own slice (and rank 0 all of them)
    def feats_of(rows_lo, rows_hi):
        gi = torch.arange(rows_lo, rows_hi, device=dev, dtype=torch.float32)
        ch = torch.arange(c, device=dev, dtype=torch.float32)
        return torch.sin(gi[:, None] * 0.37 + ch[None, :] * 1.3).to(dt)
    owned = feats_of(lo, hi)

    def step():
        return partitioned_conv(owned, w, plan)

    for _ in range(3):
        out = step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ex_ms = conv_ms = 0.0
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(args.iters):
        out = step()
    e.record()
    torch.cuda.synchronize()
    total_ms = torch.tensor([s.elapsed_time(e) / args.iters], device=dev, dtype=torch.float64)
    # exchange alone
    s.record()
    for _ in range(args.iters):
        plan.exchange(owned)
    e.record()
    torch.cuda.synchronize()
    ex = torch.tensor([s.elapsed_time(e) / args.iters], device=dev, dtype=torch.float64)
    halo = torch.tensor([plan.num_halo], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(total_ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(ex, op=dist.ReduceOp.MAX)
        dist.all_reduce(halo, op=dist.ReduceOp.SUM)
    check_device_status(dev)

    max_diff = None
    if args.check:
        outs = [torch.empty((bounds[r + 1] - bounds[r], c), dtype=dt, device=dev) for r in range(world)]
        if world > 1:
            for r in range(world):  # gather every rank's rows on rank 0 (equal-count ranges differ by at most one row)
                buf = out if r == rank else outs[r]
                dist.broadcast(buf, src=r)
                outs[r] = buf
        else:
            outs = [out]
        if rank == 0:
            km = generate_kernel_map(gc, gc, (1, 1, 1), (3, 3, 3))
            full = sparse_conv_fused(feats_of(0, n), w, km, n)
            got = torch.cat(outs, 0)
            max_diff = float((full.float() - got.float()).abs().max())
    if rank == 0:
        print(json.dumps({
            "workload": "3x3x3 stride-1 conv on one LiDAR scene split by Morton range", "n_gpus": world, "voxels": n,
            "scene": info, "channels": c, "dtype": args.dtype, "ms_per_conv": float(total_ms), "ms_exchange": float(ex),
            "voxels_per_s": n / float(total_ms) * 1e3, "halo_rows_total": int(halo.item()),
            "halo_fraction": float(halo.item()) / n, "max_abs_diff_vs_single_gpu": max_diff}), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
