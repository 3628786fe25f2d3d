"""One large outdoor scene split across GPUs by Morton-code range: a 3x3x3 stride-1
convolution with a one-voxel NCCL halo exchange that overlaps the interior rows.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m warpconvnet_b200.examples.partitioned_conv_bench --voxels 8000000 --channels 128 --dtype bf16

Rank 0 builds the seeded synthetic LiDAR scene and broadcasts its coordinates; every rank
sorts them by Morton code, owns an equal-count range, plans its halo once, then times the
convolution (exchange on its own stream + interior rows, then boundary rows) with CUDA events;
the slowest rank counts.  Rank 0 prints one JSON line; with --check the whole scene is also
run on rank 0 alone and compared with the ranks' rows bit for bit.
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


def shared_scene(voxels: int, sweeps: int, azimuth_steps: int, dev, rank: int, world: int):
    """Batch-indexed coordinates of the scene on every rank; generated once, on rank 0."""
    info = None
    if rank == 0:
        xyz, info = synthetic.lidar_scene(voxels, sweeps, azimuth_steps, seed=500)
        coords = torch.from_numpy(np.concatenate([np.zeros((len(xyz), 1), np.int32), xyz], 1)).to(dev)
        n = torch.tensor([len(xyz)], device=dev, dtype=torch.int64)
    else:
        n = torch.zeros(1, device=dev, dtype=torch.int64)
    if world > 1:
        dist.broadcast(n, src=0)
        if rank != 0:
            coords = torch.empty((int(n.item()), 4), dtype=torch.int32, device=dev)
        dist.broadcast(coords, src=0)
    return coords, info


def _features(rows_lo: int, rows_hi: int, c: int, dt, dev):
    """Features as a function of the global row, so that every rank can make its own slice."""
    gi = torch.arange(rows_lo, rows_hi, device=dev, dtype=torch.float32)
    ch = torch.arange(c, device=dev, dtype=torch.float32)
    return torch.sin(gi[:, None] * 0.37 + ch[None, :] * 1.3).to(dt)


def measure(coords: torch.Tensor, channels: int, dtype: torch.dtype, iters: int, rank: int, world: int, check: bool = False):
    """Times of the partitioned convolution over ``coords`` (the same on every rank); a dict on
    every rank (maxima / sums over ranks already taken)."""
    dev = coords.device
    n = coords.shape[0]
    perm, bounds = morton_partition(coords, world)
    gc = coords[perm].contiguous()
    plan = plan_halo(gc, bounds, rank, world)
    lo, hi = bounds[rank], bounds[rank + 1]
    c = channels
    g = torch.Generator(device="cpu").manual_seed(1)
    w = ((torch.rand(27, c, c, generator=g) * 2 - 1) * (3.0 / (27 * c)) ** 0.5 * 1.73).to(dev, dtype)
    local = plan.new_local(c, dtype, dev)
    local[:plan.num_owned] = _features(lo, hi, c, dtype, dev)
    out = torch.empty((plan.num_owned, c), dtype=dtype, device=dev)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(iters):
            fn()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / iters], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ms_overlap = timed(lambda: partitioned_conv(local, w, plan, out=out))
    ms_serial = timed(lambda: partitioned_conv(local, w, plan, out=out, overlap=False))
    ms_exchange = timed(lambda: plan.exchange_into(local))
    # the convolution alone (halo rows as they are): what a rank would take with a free exchange
    from ..geometry.coords.search.search_results import IntSearchResult
    if plan.kernel_map is None:
        plan.kernel_map = IntSearchResult.from_neighbor_table(plan.nbr_local, plan.num_local, None, None)
    ms_conv = timed(lambda: sparse_conv_fused(local, w, plan.kernel_map, plan.num_owned, split_k=1))
    halo = torch.tensor([plan.num_halo, len(plan.boundary_rows) if plan.boundary_rows is not None else 0],
                        device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(halo, op=dist.ReduceOp.SUM)
    check_device_status(dev)
    res = {"n_gpus": world, "voxels": n, "channels": c, "dtype": str(dtype).replace("torch.", ""),
           "ms_per_conv": ms_overlap, "ms_per_conv_exchange_then_conv": ms_serial, "ms_exchange": ms_exchange,
           "ms_conv_alone": ms_conv, "voxels_per_s": n / ms_overlap * 1e3, "halo_rows_total": int(halo[0].item()),
           "boundary_rows_total": int(halo[1].item()), "halo_fraction": float(halo[0].item()) / n}
    if check:
        result = partitioned_conv(local, w, plan, out=out)
        outs = [torch.empty((bounds[r + 1] - bounds[r], c), dtype=dtype, device=dev) for r in range(world)]
        if world > 1:
            for r in range(world):  # every rank's rows to rank 0
                buf = result if r == rank else outs[r]
                dist.broadcast(buf, src=r)
                outs[r] = buf
        else:
            outs = [result]
        if rank == 0:
            km = generate_kernel_map(gc, gc, (1, 1, 1), (3, 3, 3))
            full = sparse_conv_fused(_features(0, n, c, dtype, dev), w, km, n, split_k=1)
            res["max_abs_diff_vs_single_gpu"] = float((full.float() - torch.cat(outs, 0).float()).abs().max())
    return res


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
    coords, info = shared_scene(args.voxels, args.sweeps, args.azimuth_steps, dev, rank, world)
    res = measure(coords, args.channels, DT[args.dtype], args.iters, rank, world, check=args.check)
    if rank == 0:
        res["workload"] = "3x3x3 stride-1 conv on one LiDAR scene split by Morton range"
        res["scene"] = info
        print(json.dumps(res), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
