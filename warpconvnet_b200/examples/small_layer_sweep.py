"""Small-layer sweep: the 3x3x3 layers of the coarse levels of a MinkUNet (a batch of synthetic rooms
strided 4x, 8x and 16x) under every launch shape of the tensor-core kernel.

    python -m warpconvnet_b200.examples.small_layer_sweep --scenes 8 --voxels 150000

For each (level, C_in, C_out) prints one JSON line with microseconds (CUDA events, L2 flushed between
iterations) per ``split_k`` value: 0 = the library's choice, 1 = one pass with its column-block
rule, -1 = one pass and one full-width CTA per tile, -2 = two column blocks, s >= 2 = the kernel
offsets of a row block divided among s CTAs plus the slice-reduction kernel.
"""
from __future__ import annotations

import argparse
import json

import torch

from .. import POINT_ORDERING, Voxels, generate_kernel_map, stride_coords
from .._native import CONV_TCGEN05, check_device_status
from ..datasets import synthetic
from ..nn.functional.sparse_conv import sparse_conv_fused

CASES = [(4, 256, 256), (4, 128, 256), (3, 128, 128), (3, 64, 128), (3, 256, 256), (3, 384, 256), (2, 64, 64),
         (2, 32, 64), (2, 128, 128), (2, 192, 128)]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--scenes", type=int, default=8)
    ap.add_argument("--voxels", type=int, default=150000)
    ap.add_argument("--voxel-size", type=float, default=0.02)
    ap.add_argument("--split-k", default="0,1,-1,-2,2,3,4,8")
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    rooms = [synthetic.room_scene(args.voxels, args.voxel_size, 200 + s, "raster_crop") for s in range(args.scenes)]
    coords, offsets = synthetic.batch_scenes(rooms)
    vox = Voxels(torch.from_numpy(coords[:, 1:].copy()).to(dev), torch.zeros(len(coords), 1, device=dev),
                 offsets=torch.from_numpy(offsets))
    levels = [vox.sort(POINT_ORDERING.MORTON_XYZ).batch_indexed_coordinates.contiguous()]
    for _ in range(4):
        levels.append(stride_coords(levels[-1], (2, 2, 2))[0].contiguous())
    maps = {i: generate_kernel_map(c, c, (1, 1, 1), (3, 3, 3)) for i, c in enumerate(levels) if i >= 2}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

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
    for level, c_in, c_out in CASES:
        kmap, n = maps[level], levels[level].shape[0]
        x = torch.randn(n, c_in, generator=g).half().to(dev)
        w = (torch.randn(27, c_in, c_out, generator=g) * 0.05).half().to(dev)
        pairs = int((kmap.neighbor_table(n) >= 0).sum())
        row = {}
        for s in [int(v) for v in args.split_k.split(",")]:
            try:
                row[str(s)] = round(time_us(lambda: sparse_conv_fused(x, w, kmap, n, algo=CONV_TCGEN05, split_k=s)), 1)
            except RuntimeError:
                row[str(s)] = None  # a column-block count this width does not divide into
        check_device_status(dev)
        print(json.dumps({"rows": n, "tiles": (n + 127) // 128, "c_in": c_in, "c_out": c_out, "pairs_per_row": pairs / n,
                          "us_by_split_k": row, "useful_tflops_auto": 2.0 * pairs * c_in * c_out / row["0"] / 1e6}),
              flush=True)


if __name__ == "__main__":
    main()
