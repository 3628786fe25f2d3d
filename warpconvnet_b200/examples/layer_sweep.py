"""Single-layer sweep of the sparse convolution: one synthetic room, kernel 3x3x3
stride 1, 2x2x2 stride-2 down-sampling and 2x2x2 transposed up-sampling, for
C_in = C_out in a list of widths and fp16 / bf16 features with fp32 accumulation.

    python -m warpconvnet_b200.examples.layer_sweep --voxels 500000 --voxel-size 0.01

Prints one JSON line per case: milliseconds (CUDA events, L2 flushed between
iterations), useful TFLOP/s (2 * pairs * C_in * C_out / t; zero-filled rows do not
count), algorithmic GB/s, the binding roofline and the fraction of it.
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np
import torch

from .. import POINT_ORDERING, Voxels, generate_kernel_map, stride_coords
from .._native import CONV_AUTO, CONV_SIMT, CONV_TCGEN05, check_device_status
from ..datasets import synthetic
from ..nn.functional.sparse_conv import ConvEpilogue, sparse_conv_fused, sparse_conv_wgrad

DT = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}
ALGOS = {"auto": CONV_AUTO, "simt": CONV_SIMT, "tcgen05": CONV_TCGEN05}


def peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                        "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


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


def measure(voxels: int = 500000, voxel_size: float = 0.01, mode: str = "raster_crop", channels=(32, 64, 128, 256),
            dtypes=("fp16", "bf16"), kinds=("conv3", "down2", "up2"), algo: str = "auto", iters: int = 10,
            sort: bool = True, dev=None, flush=None, residual: bool = False):
    """One dict per (kind, width, dtype) case of the single-layer sweep."""
    dev = dev or torch.device("cuda", 0)
    hbm, tflops, src = peaks()
    xyz = synthetic.room_scene(voxels, voxel_size, 100, mode)
    n = len(xyz)
    vox = Voxels(torch.from_numpy(xyz).to(dev), torch.zeros(n, 1, device=dev), offsets=torch.tensor([0, n]))
    if sort:
        vox = vox.sort(POINT_ORDERING.MORTON_XYZ)
    fine = vox.batch_indexed_coordinates.contiguous()
    coarse, _ = stride_coords(fine, (2, 2, 2))
    maps = {
        "conv3": (generate_kernel_map(fine, fine, (1, 1, 1), (3, 3, 3)), n, n),
        "down2": (generate_kernel_map(fine, coarse, (2, 2, 2), (2, 2, 2)), n, len(coarse)),
    }
    maps["up2"] = (maps["down2"][0].swapped(num_in=n), len(coarse), n)
    # the coarse set is the strided fine set: every fine voxel has one parent and one offset, which is what
    # generate_output_coords_and_kernel_map records on such a map (under `auto` the layer then runs from the input side)
    maps["up2"][0]._one_pair = True
    if flush is None:
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    g = torch.Generator(device="cpu").manual_seed(0)
    lines = []
    for kind_arg in kinds:
        kind, _, which = kind_arg.partition(":")
        kmap, n_in, n_out = maps[kind]
        nbr = kmap.neighbor_table(n_out)
        pairs = int((nbr >= 0).sum().item())
        K = nbr.shape[0]
        for c in channels:
            for dname in dtypes:
                dt = DT[dname]
                x = torch.randn(n_in, c, generator=g).to(dev, dt)
                bound = (3.0 / (K * c)) ** 0.5 * 1.73
                w = ((torch.rand(K, c, c, generator=g) * 2 - 1) * bound).to(dev, dt)
                if which == "dw":    # weight gradient: X^T dY over the rows, one launch
                    gy = torch.randn(n_out, c, generator=g).to(dev, dt)
                    fn = lambda: sparse_conv_wgrad(x, gy, kmap, n_out)
                elif which == "dx":  # input gradient: the forward kernel over the transposed table
                    gy = torch.randn(n_out, c, generator=g).to(dev, dt)
                    wt, kt = w.transpose(1, 2).contiguous(), kmap.swapped(num_in=n_in)
                    fn = lambda: sparse_conv_fused(gy, wt, kt, n_in, algo=ALGOS[algo])
                elif residual:  # the second convolution of a residual block: folded BatchNorm, + identity, ReLU
                    ep = ConvEpilogue(scale=torch.rand(c, generator=g).to(dev) + 0.5, shift=torch.randn(c, generator=g).to(dev),
                                      residual=torch.randn(n_out, c, generator=g).to(dev, dt), relu=True)
                    fn = lambda: sparse_conv_fused(x, w, kmap, n_out, epilogue=ep, algo=ALGOS[algo])
                else:
                    fn = lambda: sparse_conv_fused(x, w, kmap, n_out, algo=ALGOS[algo])
                ms = time_ms(fn, iters, flush)
                check_device_status(dev)
                es = 4 if dt == torch.float32 else 2
                flop = 2.0 * pairs * c * c
                byts = es * (n_in * c + n_out * c * (2 if residual and not which else 1) + K * c * c) + 4.0 * n_out * K
                t_tc, t_hbm = flop / (tflops * 1e12), byts / (hbm * 1e9)
                lines.append({
                    "kind": kind_arg + ("+residual" if residual and not which else ""), "c": c, "dtype": dname, "voxels_in": n_in, "voxels_out": n_out, "pairs": pairs,
                    "pairs_per_out": pairs / n_out, "ms": ms, "useful_tflops": flop / ms / 1e9,
                    "alg_gbs": byts / ms / 1e6, "bound": "tensor" if t_tc > t_hbm else "hbm",
                    "roofline_frac": max(t_tc, t_hbm) / (ms * 1e-3), "peaks": src,
                    "mvoxels_per_s": n_in / ms / 1e3})
    return lines


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--voxels", type=int, default=500000)
    ap.add_argument("--voxel-size", type=float, default=0.01)
    ap.add_argument("--mode", default="raster_crop")
    ap.add_argument("--channels", default="32,64,128,256")
    ap.add_argument("--dtypes", default="fp16,bf16")
    ap.add_argument("--kinds", default="conv3,down2,up2",
                    help="conv3, down2, up2 (forward); append :dx or :dw for the two backward launches, e.g. conv3:dw")
    ap.add_argument("--algo", default="auto", choices=list(ALGOS))
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--no-sort", action="store_true", help="keep the generator's random row order")
    ap.add_argument("--residual", action="store_true",
                    help="forward layers carry the tail of a residual block: scale/shift, + residual rows, ReLU")
    args = ap.parse_args()
    lines = measure(args.voxels, args.voxel_size, args.mode, [int(v) for v in args.channels.split(",")],
                    args.dtypes.split(","), args.kinds.split(","), args.algo, args.iters, not args.no_sort,
                    residual=args.residual)
    for line in lines:
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
