"""Generate the golden fixtures in this folder FROM THE REFERENCE ITSELF.

Run on a machine that has the reference tree (its location is taken from the
environment variable ``WCN_REFERENCE_ROOT``):

    python tests/golden/make_golden.py

Sources of the stored answers:
* kernel offsets, explicit-GEMM convolution outputs and module weight init: the
  reference's own Python functions, imported with its GPU-only dependencies
  stubbed and run on CPU tensors;
* hash search, kernel maps (found -> compacted), Morton codes: the reference's
  own kernel sources compiled as host C++ (``oracle/ref_build.py``).
Inputs are seeded NumPy arrays and are stored next to the answers.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import kernel_map as km  # noqa: E402
from oracle import ref_build, ref_loader  # noqa: E402
from warpconvnet_b200.datasets import synthetic  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def batched_cloud(rng, n_per_batch, lo, hi):
    rows = []
    for b, n in enumerate(n_per_batch):
        span = hi - lo
        cells = rng.choice(span**3, n, replace=False)
        xyz = np.stack(np.unravel_index(cells, (span, span, span)), 1).astype(np.int32) + lo
        rows.append(np.concatenate([np.full((n, 1), b, np.int32), xyz], 1))
    return np.concatenate(rows, 0)


def main():
    ref_build.build(force=True)
    ref = ref_loader.import_reference_python()
    if sys.argv[1:] == ["extra"]:  # only the newer fixture; the others stay byte-identical
        extra(ref)
        return
    rng = np.random.default_rng(1234)

    # 1. kernel offsets
    np.savez_compressed(
        os.path.join(OUT, "kernel_offsets.npz"),
        k333=ref.kernel_offsets_from_size((3, 3, 3), (1, 1, 1)).numpy(),
        k222=ref.kernel_offsets_from_size((2, 2, 2), (1, 1, 1)).numpy(),
        k312=ref.kernel_offsets_from_size((3, 1, 2), (1, 1, 1)).numpy(),
        k333_d2=ref.kernel_offsets_from_size((3, 3, 3), (2, 2, 2)).numpy(),
    )

    # 2. hash search + kernel maps on a ragged 3-item batch with negative coordinates
    coords = batched_cloud(rng, [1500, 37, 900], -9, 9)
    table = ref_loader.RefHashTable(coords, "city")
    absent = coords[rng.choice(len(coords), 400)] + np.array([0, 40, 0, 0], np.int32)
    queries = np.concatenate([coords[rng.choice(len(coords), 400)], absent], 0)
    search = table.search(queries)
    in333, out333, off333 = ref_loader.ref_generate_kernel_map(coords, coords, (1, 1, 1), (3, 3, 3))
    out_coords, _ = km.stride_coords(coords, (2, 2, 2))
    in222, out222, off222 = ref_loader.ref_generate_kernel_map(coords, out_coords, (2, 2, 2), (2, 2, 2))
    # transposed: table on the fine coordinates, coarse * stride as queries (sparse_conv.py:1945-1958)
    fin, fout, foff = ref_loader.ref_generate_kernel_map(coords, out_coords, (2, 2, 2), (2, 2, 2))
    in312, out312, off312 = ref_loader.ref_generate_kernel_map(coords, coords, (1, 1, 1), (3, 1, 2))
    np.savez_compressed(
        os.path.join(OUT, "kmap_small.npz"), coords=coords, queries=queries, search=search,
        in333=in333, out333=out333, off333=off333, out_coords=out_coords,
        in222=in222, out222=out222, off222=off222,
        tr_in=fout, tr_out=fin, tr_off=foff,   # swapped: in = coarse rows, out = fine rows
        in312=in312, out312=out312, off312=off312,
        morton_xyz=coords[:, 1:] - coords[:, 1:].min(0), morton=ref_loader.ref_morton20(
            np.ascontiguousarray(coords[:, 1:] - coords[:, 1:].min(0))),
    )

    # 3. small convolutions, full tensors, fp32
    torch.manual_seed(7)
    N = len(coords)
    x = torch.randn(N, 8)
    w333 = torch.randn(27, 8, 12) * 0.2
    w222 = torch.randn(8, 8, 12) * 0.2
    wtr = torch.randn(8, 12, 8) * 0.2
    km333 = ref.IntSearchResult(torch.from_numpy(in333), torch.from_numpy(out333), torch.from_numpy(off333), 13)
    y333 = ref.explicit_gemm_forward(x, w333, km333, N)
    km222 = ref.IntSearchResult(torch.from_numpy(in222), torch.from_numpy(out222), torch.from_numpy(off222), None)
    y222 = ref.explicit_gemm_forward(x, w222, km222, len(out_coords))
    kmtr = ref.IntSearchResult(torch.from_numpy(fout), torch.from_numpy(fin), torch.from_numpy(foff), None)
    ytr = ref.explicit_gemm_forward(y222, wtr, kmtr, N)
    np.savez_compressed(os.path.join(OUT, "conv_small.npz"), x=x.numpy(), w333=w333.numpy(), y333=y333.numpy(),
                        w222=w222.numpy(), y222=y222.numpy(), wtr=wtr.numpy(), ytr=ytr.numpy())

    # 4. config 1: 20 000 voxels of [0,64)^3, C=32, fp32, reference module init
    xyz = synthetic.random_cells(20000, 64, seed=0)
    c1 = np.concatenate([np.zeros((len(xyz), 1), np.int32), xyz], 1)
    x1 = np.random.default_rng(0).standard_normal((20000, 32)).astype(np.float32)
    torch.manual_seed(0)
    mod = ref.SpatiallySparseConv(32, 32, 3, bias=False)
    w1 = mod.weight.detach().clone()
    i1, o1, f1 = ref_loader.ref_generate_kernel_map(c1, c1, (1, 1, 1), (3, 3, 3))
    km1 = ref.IntSearchResult(torch.from_numpy(i1), torch.from_numpy(o1), torch.from_numpy(f1), 13)
    y1 = ref.explicit_gemm_forward(torch.from_numpy(x1), w1, km1, len(c1)).numpy()
    rows = np.arange(0, 20000, 50)
    np.savez_compressed(
        os.path.join(OUT, "conv_config1.npz"), weight=w1.numpy(), rows=rows, y_rows=y1[rows],
        y_colsum=y1.astype(np.float64).sum(0), y_sqnorm=np.array((y1.astype(np.float64) ** 2).sum()),
        offsets=f1, in_maps_sum=np.array(i1.astype(np.int64).sum()), out_maps_sum=np.array(o1.astype(np.int64).sum()),
        weight_bound=np.array(float(w1.abs().max())),
    )
    extra(ref)
    for f in sorted(os.listdir(OUT)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(OUT, f)))


def extra(ref):
    """kmap_extra.npz: dilated and re-centred kernel maps (the reference's offset-list kernel),
    the output support of a generative convolution (its expand_coords with its own search kernel)
    and window reductions (its to_csr + row_reduction)."""
    rng = np.random.default_rng(4321)
    coords = batched_cloud(rng, [700, 25, 500], -7, 7)
    dil, ctr = (2, 1, 3), (0, 1, 2)
    offs_d = ref.kernel_offsets_from_size((3, 3, 3), dil).numpy()
    offs_c = ref.kernel_offsets_from_size((3, 2, 3), (1, 1, 1), center_offset=ctr).numpy()
    found_d = ref_loader.ref_kernel_map_found_offsets(coords, coords, (1, 1, 1), offs_d)
    found_c = ref_loader.ref_kernel_map_found_offsets(coords, coords, (1, 1, 1), offs_c)
    coarse, _ = km.stride_coords(coords, (2, 2, 2))
    found_ds = ref_loader.ref_kernel_map_found_offsets(coords, coarse, (2, 2, 2), offs_d)
    offs_e = ref.kernel_offsets_from_size((3, 3, 3), (1, 2, 1)).numpy()
    grown = ref_loader.ref_expand_coords(coords, offs_e, kernel_batch=9)  # 27 // kernel_size[0], expand.py:28-29
    # pooling over the 2x2x2 stride-2 map: the reference's CSR form and row_reduction
    i222, o222, f222 = ref_loader.ref_generate_kernel_map(coords, coarse, (2, 2, 2), (2, 2, 2))
    kmap = ref.IntSearchResult(torch.from_numpy(i222), torch.from_numpy(o222), torch.from_numpy(f222), None)
    in_csr, uniq_out, splits = kmap.to_csr()
    feats = torch.from_numpy(rng.standard_normal((len(coords), 6)).astype(np.float32))
    pooled = {}
    for red in ("max", "min", "mean", "sum", "mul", "var", "std"):
        out = torch.zeros(len(coarse), 6)
        out[uniq_out.long()] = ref.row_reduction(feats[in_csr.long()], splits, red)  # sparse_pool.py:87-104
        pooled["pool_" + red] = out.numpy()
    np.savez_compressed(
        os.path.join(OUT, "kmap_extra.npz"), coords=coords, coarse=coarse, dilation=np.array(dil), center=np.array(ctr),
        offs_d=offs_d, offs_c=offs_c, found_d=found_d, found_c=found_c, found_ds=found_ds, grown=grown,
        in222=i222, out222=o222, off222=f222, feats=feats.numpy(), **pooled)


if __name__ == "__main__":
    main()
