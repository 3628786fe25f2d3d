"""Kernel-map build alone: a batch of synthetic rooms; hash table, 3x3x3 stride-1
map, stride-2 coordinates + 2x2x2 stride-2 map and the matching transposed map.

    python -m warpconvnet_b200.examples.kernel_map_bench --scenes 4 --voxels 250000

Prints one JSON line per stage: milliseconds (CUDA events, L2 flushed between
iterations), query Mcoords/s, algorithmic GB/s (32 B per inserted key;
16 + 8 K + 24 L/M bytes per query for a K-offset map with L pairs) and its
fraction of the HBM copy bandwidth.  With --sort the rooms are Morton-ordered first
(``Voxels.sort``, timed as its own stage) and the maps come from the brick table; every map
stage includes building the tables it searches.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from .. import POINT_ORDERING, TorchHashTable, Voxels, generate_kernel_map, stride_coords
from .._native import check_device_status
from ..datasets import synthetic


def hbm_peak():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                        "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def time_ms(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        total += s.elapsed_time(e)
    return total / iters


def measure(scenes: int = 4, voxels: int = 250000, voxel_size: float = 0.02, mode: str = "raster_crop",
            iters: int = 10, sort: bool = False, dev=None, flush=None):
    """One dict per stage of the kernel-map build over a batch of synthetic rooms."""
    dev = dev or torch.device("cuda", 0)
    hbm, src = hbm_peak()
    rooms = [synthetic.room_scene(voxels, voxel_size, 100 + s, mode) for s in range(scenes)]
    coords, offsets = synthetic.batch_scenes(rooms)
    fine = torch.from_numpy(coords).to(dev)
    n = fine.shape[0]
    if flush is None:
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    origin = None
    sort_ms = None
    if sort:
        v = Voxels(fine[:, 1:].contiguous(), torch.zeros(len(fine), 1, device=dev), offsets=torch.from_numpy(offsets))
        sort_ms = time_ms(lambda: v.sort(POINT_ORDERING.MORTON_XYZ), iters, flush)
        ordered = v.sort(POINT_ORDERING.MORTON_XYZ).batched_coordinates
        fine, origin = ordered.batch_indexed_coordinates.contiguous(), ordered.morton_origin
    coarse, _ = stride_coords(fine, (2, 2, 2))
    m2 = coarse.shape[0]
    lines = []

    def report(stage, ms, queries, byts, extra=None):
        line = {"stage": stage, "generator": mode, "order": "morton" if sort else "generator", "ms": ms,
                "mcoords_per_s": queries / ms / 1e3,
                "alg_bytes": byts, "alg_gbs": byts / ms / 1e6, "hbm_frac": byts / ms / 1e6 / hbm, "peak": src,
                "queries": queries}
        line.update(extra or {})
        lines.append(line)

    if sort_ms is not None:
        report("morton_sort", sort_ms, n, 12.0 * n + 8.0 * n + 2 * 16.0 * n)
    ms = time_ms(lambda: TorchHashTable.from_keys(fine), iters, flush)
    report("hash_build", ms, n, 32.0 * n)
    if sort:
        from ..geometry.coords.search.brick_table import BrickTable
        ht0 = TorchHashTable.from_keys(fine)
        ms = time_ms(lambda: BrickTable(fine, origin, ht0), iters, flush)
        hdr = BrickTable(fine, origin, ht0).header()
        report("brick_build", ms, n, 16.0 * n + 32.0 * hdr["num_bricks"], {"bricks": hdr["num_bricks"], "usable": hdr["valid"]})

    def build_map(inc, outc, stride, ks):
        """Tables + dense neighbour table, as a forward pass builds them for one level."""
        if not sort:
            return generate_kernel_map(inc, outc, stride, ks)
        from ..geometry.coords.search.brick_table import BrickTable
        bt = BrickTable(inc, origin)  # with its stand-by voxel table: filled only if the bricks are unusable
        return generate_kernel_map(inc, outc, stride, ks, hashtable=bt.hashtable, bricks=bt)

    def full_map(inc, outc, stride, ks):
        km = build_map(inc, outc, stride, ks)
        return km.in_maps, km  # forces the compact form too

    for name, inc, outc, stride, ks in (("map_3x3x3_s1", fine, fine, (1, 1, 1), (3, 3, 3)),
                                        ("map_2x2x2_s2", fine, coarse, (2, 2, 2), (2, 2, 2))):
        K = ks[0] * ks[1] * ks[2]
        _, km = full_map(inc, outc, stride, ks)
        L, M = int(km.offsets[-1]), outc.shape[0]
        byts = 32.0 * inc.shape[0] + 16.0 * M + 8.0 * K * M + 24.0 * L + 4.0 * (K + 1)
        ms = time_ms(lambda: full_map(inc, outc, stride, ks), iters, flush)
        report(name + "_compact", ms, M, byts, {"pairs": L, "pairs_per_query": L / M})
        ms = time_ms(lambda: build_map(inc, outc, stride, ks), iters, flush)
        report(name + "_dense_only", ms, M, byts, {"pairs": L, "pairs_per_query": L / M})
    ms = time_ms(lambda: stride_coords(fine, (2, 2, 2)), iters, flush)
    report("stride_coords_2", ms, n, 16.0 * n + 32.0 * n + 16.0 * m2, {"out": m2})
    down = generate_kernel_map(fine, coarse, (2, 2, 2), (2, 2, 2))
    ms = time_ms(lambda: down.swapped(num_in=n).neighbor_table(n), iters, flush)
    report("transposed_from_forward", ms, n, 4.0 * 8 * (m2 + n))
    # tile order of the 3x3x3 table: read it twice (masks, copy), write it once, plus the row order
    km3 = generate_kernel_map(fine, fine, (1, 1, 1), (3, 3, 3))

    def tile_order():
        km3._tiled = None
        return km3.tiled_neighbor_table(n)

    ms = time_ms(tile_order, iters, flush)
    report("tile_order_3x3x3", ms, n, 4.0 * 27 * n * 3 + 8.0 * n)
    check_device_status(dev)
    return lines


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--scenes", type=int, default=4)
    ap.add_argument("--voxels", type=int, default=250000)
    ap.add_argument("--voxel-size", type=float, default=0.02)
    ap.add_argument("--mode", default="raster_crop")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--sort", action="store_true", help="Morton-sort the voxels first")
    args = ap.parse_args()
    for line in measure(args.scenes, args.voxels, args.voxel_size, args.mode, args.iters, args.sort):
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
