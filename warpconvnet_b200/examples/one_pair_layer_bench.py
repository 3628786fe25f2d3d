"""Layers in which every output row has one (input row, offset) pair, timed from both sides:
the 1x1x1 projection, the 2x2x2 stride-2 transposed convolution and the classification head of a
MinkUNet decoder on a batch of synthetic rooms.

    python -m warpconvnet_b200.examples.one_pair_layer_bench --scenes 8 --voxels 150000

One JSON line per layer: microseconds of the input-side kernel (``wcn_conv_rows_fwd``: TMA row
tiles, resident weights, scatter epilogue) and of the output-side kernels (``wcn_conv_fwd``), CUDA
events with L2 flushed between iterations, and the input-side kernel's algorithmic bytes (feature
rows read once, output rows written once, destination table, weights) against the HBM peak.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from .. import POINT_ORDERING, Voxels, generate_kernel_map, stride_coords
from .._native import CONV_TCGEN05, check_device_status
from ..datasets import synthetic
from ..geometry.coords.search.search_results import IntSearchResult
from ..nn.functional.sparse_conv import _identity_map, sparse_conv_fused, sparse_conv_rows_fused

# (kind, level of the OUTPUT rows, C_in, C_out): the decoder of MinkUNet-34 (planes 256, 128, 96, 96)
CASES = [("project", 0, 128, 96), ("up", 0, 96, 96), ("head", 0, 96, 20), ("project", 1, 128, 96), ("up", 1, 128, 96),
         ("project", 2, 192, 128), ("up", 2, 256, 128), ("up", 3, 256, 256)]


def hbm_peak_gbs() -> float:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"])
    except (OSError, KeyError, ValueError):
        return 6650.0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--scenes", type=int, default=8)
    ap.add_argument("--voxels", type=int, default=150000)
    ap.add_argument("--voxel-size", type=float, default=0.02)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--kinds", default="project,up,head")
    ap.add_argument("--levels", default="0,1,2,3")
    ap.add_argument("--skip-output-side", action="store_true", help="time the input-side kernel only")
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    rooms = [synthetic.room_scene(args.voxels, args.voxel_size, 200 + s, "raster_crop") for s in range(args.scenes)]
    coords, offsets = synthetic.batch_scenes(rooms)
    vox = Voxels(torch.from_numpy(coords[:, 1:].copy()).to(dev), torch.zeros(len(coords), 1, device=dev),
                 offsets=torch.from_numpy(offsets)).sort(POINT_ORDERING.MORTON_XYZ)
    levels = [vox.batch_indexed_coordinates.contiguous()]
    for _ in range(4):
        levels.append(stride_coords(levels[-1], (2, 2, 2))[0].contiguous())
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    peak = hbm_peak_gbs()

    def time_us(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(args.iters):
            flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            total += s.elapsed_time(e)
        return total / args.iters * 1e3

    g = torch.Generator().manual_seed(0)
    kinds, wanted = args.kinds.split(","), [int(v) for v in args.levels.split(",")]
    for kind, level, c_in, c_out in CASES:
        if kind not in kinds or level not in wanted:
            continue
        n_out = levels[level].shape[0]
        if kind == "up":
            n_in = levels[level + 1].shape[0]
            down = generate_kernel_map(levels[level], levels[level + 1], (2, 2, 2), (2, 2, 2))
            dst = down.neighbor_table(n_in)          # [8, coarse]: the child of every (parent, offset)
            out_side = down.swapped(num_in=n_out)    # the transposed map the output-side kernel reads
            K = 8
        elif kind == "head":                         # writes through the permutation of the Morton sort
            n_in, K = n_out, 1
            dst = torch.randperm(n_out, generator=g).to(torch.int32).view(1, -1).to(dev)
            inverse = torch.empty(n_out, dtype=torch.int32, device=dev)
            inverse[dst.view(-1).long()] = torch.arange(n_out, dtype=torch.int32, device=dev)
            out_side = IntSearchResult.from_neighbor_table(inverse.view(1, -1), n_out, None, None)
        else:
            n_in, K, dst = n_out, 1, None
            out_side = IntSearchResult.from_neighbor_table(_identity_map(n_out, dev).neighbor_table(n_out), n_out, None, 0)
        x = torch.randn(n_in, c_in, generator=g).half().to(dev)
        w = (torch.randn(K, c_in, c_out, generator=g) * 0.05).half().to(dev)
        t_in = time_us(lambda: sparse_conv_rows_fused(x, w, dst, n_out))
        t_out = None if args.skip_output_side else time_us(lambda: sparse_conv_fused(x, w, out_side, n_out))
        got = sparse_conv_rows_fused(x, w, dst, n_out)
        assert got is not None
        byts = 2.0 * n_in * c_in + 2.0 * n_out * c_out + (4.0 * K * n_in if dst is not None else 0.0) + 2.0 * K * c_in * c_out
        line = {"kind": kind, "rows_in": n_in, "rows_out": n_out, "offsets": K, "c_in": c_in, "c_out": c_out,
                "input_side_us": round(t_in, 1), "output_side_us": round(t_out, 1) if t_out is not None else None,
                "alg_bytes": byts, "alg_gbs": byts / t_in / 1e3, "hbm_frac": byts / t_in / 1e3 / peak}
        if t_out is not None:
            ref = sparse_conv_fused(x, w, out_side, n_out)
            line["max_abs_diff"] = float((got.float() - ref.float()).abs().max())
        check_device_status(dev)
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
