"""GPU parity of the sparse convolution through the public surface: fp32 within 1e-4
relative L2 of the reference's explicit-GEMM path, fp16/bf16 within 1e-2."""
import numpy as np
import pytest
import torch
import torch.nn as nn

from oracle import kernel_map as km
from oracle import sparse_conv as osc
from warpconvnet_b200 import (SPARSE_CONV_FWD_ALGO_MODE as ALGO, ConvEpilogue, IntSearchResult, Sequential,
                              SparseConv3d, Voxels, generate_kernel_map, spatially_sparse_conv, stride_coords)
from warpconvnet_b200._native import CONV_SIMT, CONV_TCGEN05, check_device_status
from warpconvnet_b200.datasets import synthetic
from warpconvnet_b200.examples.mink_unet import MinkUNet18, randomize_batchnorm_
from warpconvnet_b200.nn.functional.sparse_conv import sparse_conv_fused

from conftest import rel_l2

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {torch.float32: 1e-4, torch.float16: 1e-2, torch.bfloat16: 1e-2}


def make_voxels(coords_b, feats, **kw):
    offsets = np.concatenate([[0], np.cumsum(np.bincount(coords_b[:, 0]))])
    return Voxels(torch.from_numpy(coords_b[:, 1:].copy()).to(DEV), feats.to(DEV), offsets=torch.from_numpy(offsets), **kw)


@pytest.mark.parametrize("algo", [ALGO.EXPLICIT_GEMM, ALGO.IMPLICIT_GEMM, ALGO.CUTLASS_IMPLICIT_GEMM, ALGO.AUTO])
def test_small_golden_fp32(golden, algo):
    g, c = golden("kmap_small.npz"), golden("conv_small.npz")
    x = make_voxels(g["coords"], torch.from_numpy(c["x"]))
    y = spatially_sparse_conv(x, torch.from_numpy(c["w333"]).to(DEV), 3, fwd_algo=algo)
    assert rel_l2(y.feature_tensor.cpu().numpy(), c["y333"]) < 1e-4
    assert y.tensor_stride == (1, 1, 1) and torch.equal(y.coordinate_tensor, x.coordinate_tensor)
    down = spatially_sparse_conv(x, torch.from_numpy(c["w222"]).to(DEV), 2, stride=2, fwd_algo=algo)
    assert down.tensor_stride == (2, 2, 2)
    assert np.array_equal(down.batch_indexed_coordinates.cpu().numpy(), g["out_coords"])
    assert rel_l2(down.feature_tensor.cpu().numpy(), c["y222"]) < 1e-4
    up = spatially_sparse_conv(down, torch.from_numpy(c["wtr"]).to(DEV), 2, stride=2, transposed=True,
                               output_spatially_sparse_tensor=x, fwd_algo=algo)
    assert up.tensor_stride == (1, 1, 1) and len(up) == len(x)
    assert rel_l2(up.feature_tensor.cpu().numpy(), c["ytr"]) < 1e-4
    assert len(x.cache) == 3  # 3x3x3 map, down map, transposed map share one cache
    check_device_status(DEV)


@pytest.mark.parametrize("algo", [ALGO.EXPLICIT_GEMM, ALGO.IMPLICIT_GEMM])
def test_config1_golden_fp32(golden, algo):
    """Single SparseConv3d layer: 20 000 voxels of [0,64)^3, C_in = C_out = 32, 3x3x3, fp32, no bias."""
    g = golden("conv_config1.npz")
    xyz = synthetic.random_cells(20000, 64, seed=0)
    coords = np.concatenate([np.zeros((len(xyz), 1), np.int32), xyz], 1)
    feats = torch.from_numpy(np.random.default_rng(0).standard_normal((20000, 32)).astype(np.float32))
    x = make_voxels(coords, feats)
    conv = SparseConv3d(32, 32, 3, bias=False, fwd_algo=algo).to(DEV)
    assert float(conv.weight.abs().max()) <= float(g["weight_bound"]) * 1.05  # same init bound as the reference
    with torch.no_grad():
        conv.weight.copy_(torch.from_numpy(g["weight"]))
        y = conv(x).feature_tensor.cpu().numpy()
    assert rel_l2(y[g["rows"]], g["y_rows"]) < 1e-4
    assert np.allclose(y.astype(np.float64).sum(0), g["y_colsum"], rtol=1e-4, atol=1e-3)
    kmap = next(iter(x.cache.values()))
    assert np.array_equal(kmap.offsets.numpy(), g["offsets"])
    assert int(kmap.in_maps.long().sum()) == int(g["in_maps_sum"])


def _layer_case(n, c_in, c_out, seed, mode="raster_crop"):
    xyz = synthetic.room_scene(n, 0.02, seed, mode)
    coords = np.concatenate([np.zeros((len(xyz), 1), np.int32), xyz], 1)
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, c_in, generator=g)
    w = (torch.rand(27, c_in, c_out, generator=g) * 2 - 1) * (3.0 / (27 * c_in)) ** 0.5 * 1.73
    return coords, x, w


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("c_in,c_out", [(32, 32), (64, 64), (96, 96), (128, 96), (128, 128), (256, 256), (384, 256),
                                        (192, 128), (32, 64), (64, 16)])
def test_tcgen05_matches_oracle(dtype, c_in, c_out):
    n = 6000 if c_in * c_out > 20000 else 12000
    coords, x, w = _layer_case(n, c_in, c_out, 400 + c_in + c_out)
    xq, wq = x.to(dtype), w.to(dtype)
    i, o, f, iden = km.generate_kernel_map(coords, coords, (1, 1, 1), (3, 3, 3))
    ref = osc.explicit_gemm_forward(xq.float(), wq.float(), i, o, f, iden, n).numpy()  # fp32 on the quantised inputs
    c = torch.from_numpy(coords).to(DEV)
    kmap = generate_kernel_map(c, c, (1, 1, 1), (3, 3, 3))
    y = sparse_conv_fused(xq.to(DEV), wq.to(DEV), kmap, n, algo=CONV_TCGEN05)
    check_device_status(DEV)
    assert y.dtype == dtype
    assert rel_l2(y.float().cpu().numpy(), ref) < TOL[dtype]
    y32 = sparse_conv_fused(xq.to(DEV), wq.to(DEV), kmap, n, out_dtype=torch.float32, algo=CONV_TCGEN05)
    assert rel_l2(y32.cpu().numpy(), ref) < 1e-4  # fp32 accumulation: only summation order differs
    ys = sparse_conv_fused(xq.to(DEV), wq.to(DEV), kmap, n, out_dtype=torch.float32, algo=CONV_SIMT)
    assert rel_l2(ys.cpu().numpy(), ref) < 1e-4
    # bit-reproducible
    y2 = sparse_conv_fused(xq.to(DEV), wq.to(DEV), kmap, n, algo=CONV_TCGEN05)
    assert torch.equal(y, y2)


def _oracle_rows(coords, xq, wq, rows):
    """Reference output for a subset of output rows (pairs restricted to those rows)."""
    found = km.kernel_map_found(coords, coords[rows], (1, 1, 1), (3, 3, 3))
    out = torch.zeros(len(rows), wq.shape[2])
    for k in range(27):
        hit = np.nonzero(found[k] >= 0)[0]
        if len(hit):
            out[torch.from_numpy(hit)] += xq[torch.from_numpy(found[k][hit]).long()] @ wq[k]
    return out.numpy()


@pytest.mark.parametrize("c_in,c_out,n", [(32, 32, 200000), (64, 64, 200000), (96, 96, 160000), (128, 128, 120000),
                                          (256, 256, 100000), (64, 128, 40000), (128, 96, 300000)])
def test_tcgen05_large_problem(c_in, c_out, n):
    """Sizes at which the kernel runs several 128-row sub-tiles per CTA pass and double-buffered
    accumulators: tensor-core kernel == FP32-pipe kernel everywhere, == oracle on row samples,
    with the fused epilogue on, and bit-reproducible."""
    coords, x, w = _layer_case(n, c_in, c_out, 900 + c_in, "raster_crop")
    order = np.argsort(km.morton_code(coords[:, 1:]), kind="stable")  # spatially coherent tiles
    coords = np.ascontiguousarray(coords[order])
    xq, wq = x.half(), w.half()
    g = torch.Generator().manual_seed(3)
    scale, shift = torch.rand(c_out, generator=g) + 0.5, torch.randn(c_out, generator=g) * 0.1
    res = torch.randn(n, c_out, generator=g).half()
    c = torch.from_numpy(coords).to(DEV)
    kmap = generate_kernel_map(c, c, (1, 1, 1), (3, 3, 3))
    ep = ConvEpilogue(scale=scale.to(DEV), shift=shift.to(DEV), residual=res.to(DEV), relu=True)
    y = sparse_conv_fused(xq.to(DEV), wq.to(DEV), kmap, n, epilogue=ep, algo=CONV_TCGEN05)
    check_device_status(DEV)
    ys = sparse_conv_fused(xq.to(DEV), wq.to(DEV), kmap, n, epilogue=ep, algo=CONV_SIMT)
    assert rel_l2(y.float().cpu().numpy(), ys.float().cpu().numpy()) < 2e-3  # both rounded to fp16
    for rows in (np.arange(0, 1500), np.arange(n - 1500, n), np.arange(n // 2, n // 2 + 1500)):
        conv = torch.from_numpy(_oracle_rows(coords, xq.float(), wq.float(), rows))
        ref = torch.relu(conv * scale + shift + res[rows].float()).numpy()
        assert rel_l2(y[rows].float().cpu().numpy(), ref) < 1e-2
    y2 = sparse_conv_fused(xq.to(DEV), wq.to(DEV), kmap, n, epilogue=ep, algo=CONV_TCGEN05)
    assert torch.equal(y, y2)


@pytest.mark.parametrize("dtype,algo,c_in,c_out", [(torch.float16, CONV_TCGEN05, 96, 96),
                                                   (torch.bfloat16, CONV_TCGEN05, 64, 128),
                                                   (torch.float32, CONV_SIMT, 24, 40)])
def test_tile_order_is_bit_identical(dtype, algo, c_in, c_out):
    """Running the output rows in tile order (grouped by neighbour pattern) changes which
    (tile, offset) pairs are computed, not one bit of the result: 3x3x3, 2x2x2 stride 2 and
    its transposed map, epilogue with residual on."""
    n = 50000
    coords, x, w = _layer_case(n, c_in, c_out, 77, "raster_crop")
    coords = np.ascontiguousarray(coords[np.argsort(km.morton_code(coords[:, 1:]), kind="stable")])
    c = torch.from_numpy(coords).to(DEV)
    coarse, _ = stride_coords(c, (2, 2, 2))
    g = torch.Generator().manual_seed(9)
    down = generate_kernel_map(c, coarse, (2, 2, 2), (2, 2, 2))
    cases = [(generate_kernel_map(c, c, (1, 1, 1), (3, 3, 3)), n, n, 27),
             (down, n, len(coarse), 8), (down.swapped(num_in=n), len(coarse), n, 8)]
    for kmap, n_in, n_out, K in cases:
        xin = torch.randn(n_in, c_in, generator=g).to(dtype).to(DEV)
        wk = (torch.randn(K, c_in, c_out, generator=g) * 0.1).to(dtype).to(DEV)
        ep = ConvEpilogue(scale=(torch.rand(c_out, generator=g) + 0.5).to(DEV),
                          shift=torch.randn(c_out, generator=g).to(DEV),
                          residual=torch.randn(n_out, c_out, generator=g).to(dtype).to(DEV), relu=True)
        a = sparse_conv_fused(xin, wk, kmap, n_out, epilogue=ep, algo=algo, tile_order=False)
        b = sparse_conv_fused(xin, wk, kmap, n_out, epilogue=ep, algo=algo, tile_order=True)
        check_device_status(DEV)
        assert torch.equal(a, b)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("c_in,c_out", [(32, 16), (64, 48), (32, 80), (96, 112), (64, 144), (128, 256)])
def test_residual_rows_of_every_width(dtype, c_in, c_out):
    """The tensor-core kernel reads the residual of 16-bit outputs through shared memory, 64 columns at a
    time with a narrower last piece: widths that end in a 16-, 32- and 48-column piece, rows in tile order
    and in table order, the residual a column block of a wider matrix and a last sub-tile that is not full.
    Against the FP32-pipe kernel (both round the same fp32 value once)."""
    n = 33333
    coords, x, w = _layer_case(n, c_in, c_out, 31 + c_out, "raster_crop")
    coords = np.ascontiguousarray(coords[np.argsort(km.morton_code(coords[:, 1:]), kind="stable")])
    c = torch.from_numpy(coords).to(DEV)
    kmap = generate_kernel_map(c, c, (1, 1, 1), (3, 3, 3))
    g = torch.Generator().manual_seed(c_out)
    wide = torch.randn(n, c_out + 32, generator=g).to(dtype).to(DEV)
    xd, wd = x.to(dtype).to(DEV), w.to(dtype).to(DEV)
    for residual in (wide[:, 16:16 + c_out], wide[:, :c_out].contiguous()):
        ep = ConvEpilogue(scale=(torch.rand(c_out, generator=g) + 0.5).to(DEV), shift=torch.randn(c_out, generator=g).to(DEV),
                          residual=residual, relu=True)
        ref = sparse_conv_fused(xd, wd, kmap, n, epilogue=ep, algo=CONV_SIMT)
        for tile_order in (False, True):
            got = sparse_conv_fused(xd, wd, kmap, n, epilogue=ep, algo=CONV_TCGEN05, tile_order=tile_order, split_k=1)
            check_device_status(DEV)
            assert rel_l2(got.float().cpu().numpy(), ref.float().cpu().numpy()) < 2e-3
            assert float((got.float() - ref.float()).abs().max()) < 0.25
        plain = sparse_conv_fused(xd, wd, kmap, n, algo=CONV_TCGEN05, split_k=1).float()
        want = torch.relu(plain * ep.scale + ep.shift + residual.float())
        assert float((got.float() - want).abs().max()) < 0.1   # `plain` is rounded once more than `got`


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("K,c_in,c_out", [(27, 3, 32), (1, 3, 32), (27, 4, 64), (8, 6, 16),
                                          (1, 96, 20), (1, 64, 8), (8, 32, 24), (1, 128, 31)])
def test_narrow_kernels_match_fp32_pipe_kernel(dtype, K, c_in, c_out):
    """Layers with a few input channels (a stem) or a few output channels (a head) take the
    streaming kernels under `auto`; they accumulate in the order of the FP32-pipe kernel, so the
    results agree bit for bit (epilogue and tile order on)."""
    from warpconvnet_b200._native import CONV_AUTO
    n = 40000
    coords, _, _ = _layer_case(n, 4, 4, 55, "raster_crop")
    coords = np.ascontiguousarray(coords[np.argsort(km.morton_code(coords[:, 1:]), kind="stable")])
    c = torch.from_numpy(coords).to(DEV)
    g = torch.Generator().manual_seed(K + c_in)
    if K == 27:
        kmap, n_out = generate_kernel_map(c, c, (1, 1, 1), (3, 3, 3)), n
    elif K == 8:
        coarse, _ = stride_coords(c, (2, 2, 2))
        kmap, n_out = generate_kernel_map(c, coarse, (2, 2, 2), (2, 2, 2)), len(coarse)
    else:
        from warpconvnet_b200.nn.functional.sparse_conv import _identity_map
        kmap, n_out = _identity_map(n, torch.device(DEV)), n
    x = torch.randn(n, c_in, generator=g).to(dtype).to(DEV)
    w = (torch.randn(K, c_in, c_out, generator=g) * 0.3).to(dtype).to(DEV)
    ep = ConvEpilogue(scale=(torch.rand(c_out, generator=g) + 0.5).to(DEV), shift=torch.randn(c_out, generator=g).to(DEV),
                      residual=torch.randn(n_out, c_out, generator=g).to(dtype).to(DEV), relu=True)
    a = sparse_conv_fused(x, w, kmap, n_out, epilogue=ep, algo=CONV_AUTO)
    b = sparse_conv_fused(x, w, kmap, n_out, epilogue=ep, algo=CONV_SIMT)
    check_device_status(DEV)
    plain = sparse_conv_fused(x, w, kmap, n_out, algo=CONV_AUTO)
    ref = sparse_conv_fused(x, w, kmap, n_out, algo=CONV_SIMT)
    if K == 1 and dtype != torch.float32 and c_in % 32 == 0:
        # 1x1x1 layers with 16-bit features run from the input side on the tensor cores under `auto`:
        # same products, fp32 sums in another order
        assert rel_l2(plain.float().cpu().numpy(), ref.float().cpu().numpy()) < 1e-3
        assert rel_l2(a.float().cpu().numpy(), b.float().cpu().numpy()) < 1e-2
        return
    assert torch.equal(plain, ref), "accumulation differs"
    assert torch.equal(a, b), "epilogue differs"


def _rows_reference(x, w, dst, n_out, scale=None, shift=None, residual=None, relu=False):
    """out[dst[k, j]] = epilogue(x[j] @ w[k]) in fp64 on the CPU (rows nobody names stay NaN)."""
    x64, w64 = x.double().cpu(), w.double().cpu()
    out = torch.full((n_out, w.shape[2]), float("nan"), dtype=torch.float64)
    for k in range(w.shape[0]):
        d = dst[k].cpu().long()
        hit = d >= 0
        out[d[hit]] = x64[hit] @ w64[k]
    if scale is not None:
        out = out * scale.double().cpu()
    if shift is not None:
        out = out + shift.double().cpu()
    if residual is not None:
        out = out + residual.double().cpu()
    return out.clamp_min(0) if relu else out


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("K,c_in,c_out", [(1, 96, 20), (1, 128, 96), (1, 32, 31), (1, 256, 256), (1, 64, 16),
                                          (8, 96, 96), (8, 128, 96), (8, 256, 128), (8, 256, 256), (8, 32, 48)])
def test_input_side_kernel_matches_fp64(dtype, K, c_in, c_out):
    """wcn_conv_rows_fwd (TMA row tiles, resident weight chunks, scatter epilogue) against an fp64
    evaluation of the same 16-bit inputs: 1x1x1 through a permutation, and the 2x2x2 stride-2 child
    table of a real scene (several weight chunks, one and two weight buffers, a ragged last tile,
    output widths that are not multiples of 16, every epilogue part)."""
    from warpconvnet_b200.nn.functional.sparse_conv import sparse_conv_rows_fused
    g = torch.Generator().manual_seed(100 * K + c_in + c_out)
    if K == 1:
        n_in = n_out = 33333
        dst = torch.randperm(n_out, generator=g).to(torch.int32).view(1, -1)
    else:
        coords, _, _ = _layer_case(60000, 4, 4, 91, "raster_crop")
        fine = torch.from_numpy(coords).to(DEV)
        coarse, _ = stride_coords(fine, (2, 2, 2))
        dst = generate_kernel_map(fine, coarse, (2, 2, 2), (2, 2, 2)).neighbor_table(len(coarse))
        n_in, n_out = len(coarse), len(fine)
        covered = torch.zeros(n_out, dtype=torch.int32, device=DEV)
        covered.index_add_(0, dst[dst >= 0].long(), torch.ones(int((dst >= 0).sum()), dtype=torch.int32, device=DEV))
        assert bool((covered == 1).all()), "every fine voxel has exactly one (parent, offset)"
    x = torch.randn(n_in, c_in, generator=g).to(dtype).to(DEV)
    w = (torch.randn(K, c_in, c_out, generator=g) * (1.0 / c_in) ** 0.5).to(dtype).to(DEV)
    dst = dst.to(DEV).contiguous()
    scale = (torch.rand(c_out, generator=g) + 0.5).to(DEV)
    shift = torch.randn(c_out, generator=g).to(DEV)
    residual = torch.randn(n_out, c_out, generator=g).to(dtype).to(DEV)
    for ep, kw in ((None, {}), (ConvEpilogue(scale=scale, shift=shift, residual=residual, relu=True),
                                dict(scale=scale, shift=shift, residual=residual, relu=True))):
        got = sparse_conv_rows_fused(x, w, dst, n_out, ep)
        assert got is not None, "the input-side kernel should take this shape"
        check_device_status(DEV)
        want = _rows_reference(x, w, dst, n_out, **kw)
        assert not torch.isnan(want).any()
        assert rel_l2(got.double().cpu().numpy(), want.numpy()) < 4e-3
    # fp32 result, feature rows and output rows inside wider buffers
    wide_in = torch.zeros(n_in, c_in + 40, dtype=dtype, device=DEV)
    wide_in[:, 8:8 + c_in] = x
    wide_out = torch.full((n_out, c_out + 24), -7.0, dtype=torch.float32, device=DEV)
    got = sparse_conv_rows_fused(wide_in[:, 8:8 + c_in], w, dst, n_out, ConvEpilogue(shift=shift, out=wide_out[:, 8:8 + c_out]),
                                 out_dtype=torch.float32)
    assert got is not None and got.data_ptr() == wide_out[:, 8:].data_ptr()
    check_device_status(DEV)
    assert rel_l2(got.double().cpu().numpy(), _rows_reference(x, w, dst, n_out, shift=shift).numpy()) < 4e-3
    assert bool((wide_out[:, :8] == -7.0).all()) and bool((wide_out[:, 8 + c_out:] == -7.0).all())


def test_transposed_stride2_takes_the_input_side_kernel_and_matches_the_output_side_one():
    """Through the public call: a 2x2x2 stride-2 transposed convolution onto the tensor it was strided
    from is tagged one-pair and runs from the input side; forcing the output-side kernel gives the
    same numbers to fp32-sum reordering."""
    coords, _, _ = _layer_case(50000, 4, 4, 17, "raster_crop")
    g = torch.Generator().manual_seed(3)
    fine = make_voxels(coords, torch.randn(len(coords), 64, generator=g).half())
    wd = (torch.randn(8, 64, 64, generator=g) * 0.1).half().to(DEV)
    wu = (torch.randn(8, 64, 96, generator=g) * 0.1).half().to(DEV)
    with torch.no_grad():
        coarse = spatially_sparse_conv(fine, wd, 2, stride=2, fwd_algo=ALGO.IMPLICIT_GEMM)
        up = spatially_sparse_conv(coarse, wu, 2, stride=2, transposed=True, output_spatially_sparse_tensor=fine,
                                   fwd_algo=ALGO.IMPLICIT_GEMM)
    kmap = [v for k, v in fine.cache.items() if k.transposed] or [v for k, v in coarse.cache.items() if k.transposed]
    assert kmap and kmap[0]._one_pair
    from warpconvnet_b200._native import LAUNCH_COUNTS
    assert LAUNCH_COUNTS["wcn_conv_rows_fwd"] >= 1
    ref = sparse_conv_fused(coarse.feature_tensor, wu, kmap[0], len(fine), algo=CONV_TCGEN05)
    check_device_status(DEV)
    assert rel_l2(up.feature_tensor.float().cpu().numpy(), ref.float().cpu().numpy()) < 1e-3


@pytest.mark.parametrize("stride", [1, 2])
def test_generative_and_dilated_convolution(stride):
    """generative=True grows the output support by the kernel window (after the stride, if any);
    dilation spaces the window.  Output rows are compared with the oracle's after sorting both
    coordinate sets (the reference defines the set, not the order)."""
    n, c_in, c_out = 4000, 8, 12
    coords, x, _ = _layer_case(n, c_in, c_out, 71, "sample")
    g = torch.Generator().manual_seed(5)
    w = torch.randn(27, c_in, c_out, generator=g) * 0.2
    vox = make_voxels(coords, x)
    dil = (1, 2, 1)
    with torch.no_grad():
        y = spatially_sparse_conv(vox, w.to(DEV), 3, stride=stride, kernel_dilation=dil, generative=True,
                                  fwd_algo=ALGO.IMPLICIT_GEMM)
    base = coords if stride == 1 else km.stride_coords(coords, (stride,) * 3)[0]
    out_c, out_off = km.expand_coords(base, (3, 3, 3), dil)
    i, o, f, iden = km.generate_kernel_map(coords, out_c, (stride,) * 3, (3, 3, 3), dil)
    want = osc.explicit_gemm_forward(x, w, i, o, f, iden, len(out_c)).numpy()
    got_c = y.batch_indexed_coordinates.cpu().numpy()
    assert len(got_c) == len(out_c) and np.array_equal(y.offsets.numpy(), out_off)
    order = np.lexsort(tuple(got_c[:, d] for d in reversed(range(4))))
    assert np.array_equal(got_c[order], out_c)
    assert rel_l2(y.feature_tensor.cpu().numpy()[order], want) < 1e-4
    check_device_status(DEV)


def test_minkunet34_is_bit_identical_with_and_without_tile_order(monkeypatch):
    """The whole network (fused epilogues, offset-spanning slots, stem and head kernels) gives the same
    bits whether the 3x3x3 layers run in tile order or in row order, and the same bits twice."""
    import warpconvnet_b200.nn.functional.sparse_conv as F
    from warpconvnet_b200 import POINT_ORDERING
    from warpconvnet_b200.examples.mink_unet import MinkUNet34
    scenes = [synthetic.room_scene(30000, 0.02, 800 + i, "raster_crop") for i in range(2)]
    coords, offsets = synthetic.batch_scenes(scenes)
    torch.manual_seed(7)
    model = MinkUNet34(3, 20).to(DEV).half().eval()
    randomize_batchnorm_(model)
    x = torch.rand(len(coords), 3, generator=torch.Generator().manual_seed(1)).half()

    def run():
        vox = Voxels(torch.from_numpy(coords[:, 1:].copy()).to(DEV), x.to(DEV), offsets=torch.from_numpy(offsets))
        with torch.no_grad():
            return model(vox.sort(POINT_ORDERING.MORTON_XYZ), restore_order=True)

    a = run()
    b = run()
    monkeypatch.setattr(F, "TILE_ORDER_MIN_ROWS", 1 << 60)
    c = run()
    check_device_status(DEV)
    assert torch.isfinite(a.float()).all() and float(a.float().abs().max()) > 0
    assert torch.equal(a, b) and torch.equal(a, c)


def test_minkunet_restore_order_equals_unpermute():
    """`restore_order=True` stores the head's rows through the sort permutation: the same
    numbers as un-permuting the sorted result afterwards."""
    from warpconvnet_b200 import POINT_ORDERING
    coords, x, _ = _layer_case(20000, 3, 4, 31, "raster_crop")
    torch.manual_seed(2)
    model = MinkUNet18(3, 20).to(DEV).half().eval()
    randomize_batchnorm_(model)
    vox = make_voxels(coords, x.half()).sort(POINT_ORDERING.MORTON_XYZ)
    perm = vox.extra_attributes["perm"]
    with torch.no_grad():
        direct = model(vox, restore_order=True)
        ref = torch.empty_like(direct)
        ref[perm] = model(vox).feature_tensor
    check_device_status(DEV)
    assert torch.equal(direct, ref)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_fused_epilogue_matches_unfused_chain(dtype):
    """conv -> BatchNorm1d(eval) -> + residual -> ReLU in one kernel vs the separate torch ops."""
    n, c_in, c_out = 9000, 64, 96
    coords, x, w = _layer_case(n, c_in, c_out, 77, "sample")
    g = torch.Generator().manual_seed(1)
    scale, shift = torch.rand(c_out, generator=g) + 0.5, torch.randn(c_out, generator=g) * 0.2
    res = torch.randn(n, c_out, generator=g)
    xq, wq, rq = x.to(dtype), w.to(dtype), res.to(dtype)
    i, o, f, iden = km.generate_kernel_map(coords, coords, (1, 1, 1), (3, 3, 3))
    conv = osc.explicit_gemm_forward(xq.float(), wq.float(), i, o, f, iden, n)
    ref = torch.relu(conv * scale + shift + rq.float()).numpy()
    c = torch.from_numpy(coords).to(DEV)
    kmap = generate_kernel_map(c, c, (1, 1, 1), (3, 3, 3))
    ep = ConvEpilogue(scale=scale.to(DEV), shift=shift.to(DEV), residual=rq.to(DEV), relu=True)
    y = sparse_conv_fused(xq.to(DEV), wq.to(DEV), kmap, n, epilogue=ep)
    assert rel_l2(y.float().cpu().numpy(), ref) < TOL[dtype]
    assert float(y.min()) >= 0.0
    check_device_status(DEV)


def test_sequential_fuses_conv_bn_relu_in_eval():
    n = 5000
    coords, x, _ = _layer_case(n, 32, 64, 91, "sample")
    vox = make_voxels(coords, x)
    torch.manual_seed(0)
    block = Sequential(SparseConv3d(32, 64, 3, bias=True), nn.BatchNorm1d(64), nn.ReLU()).to(DEV)
    randomize_batchnorm_(block, 3)
    block.eval()
    with torch.no_grad():
        fused = block(vox).feature_tensor
        conv_out = block[0](vox)
        unfused = block[2](block[1](conv_out.feature_tensor))
    assert rel_l2(fused.cpu().numpy(), unfused.cpu().numpy()) < 1e-5
    block.train()
    out_train = block(vox)  # layer by layer, batch statistics, autograd alive
    assert out_train.feature_tensor.requires_grad


def test_backward_matches_explicit_formulas():
    n = 3000
    coords, x, w = _layer_case(n, 8, 12, 13, "sample")
    i, o, f, iden = km.generate_kernel_map(coords, coords, (1, 1, 1), (3, 3, 3))
    xr, wr = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    yr = torch.zeros(n, 12)
    for k in range(27):
        s, e = int(f[k]), int(f[k + 1])
        yr = yr.index_add(0, torch.from_numpy(o[s:e]).long(), xr[torch.from_numpy(i[s:e]).long()] @ wr[k])
    go = torch.randn(n, 12, generator=torch.Generator().manual_seed(2))
    yr.backward(go)
    from warpconvnet_b200 import SPARSE_CONV_BWD_ALGO_MODE as BWD
    for algo, bwd in ((ALGO.EXPLICIT_GEMM, BWD.EXPLICIT_GEMM), (ALGO.IMPLICIT_GEMM, BWD.EXPLICIT_GEMM),
                      (ALGO.IMPLICIT_GEMM, BWD.IMPLICIT_GEMM), (ALGO.AUTO, [BWD.EXPLICIT_GEMM, BWD.CUTLASS_IMPLICIT_GEMM])):
        xg = x.clone().to(DEV).requires_grad_(True)
        wg = w.clone().to(DEV).requires_grad_(True)
        vox = make_voxels(coords, xg)
        y = spatially_sparse_conv(vox, wg, 3, fwd_algo=algo, bwd_algo=bwd)
        y.feature_tensor.backward(go.to(DEV))
        assert rel_l2(xg.grad.cpu().numpy(), xr.grad.numpy()) < 1e-4
        assert rel_l2(wg.grad.cpu().numpy(), wr.grad.numpy()) < 1e-4


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("K,c_in,c_out,n", [(27, 64, 64, 30000), (27, 128, 128, 20000), (27, 32, 32, 30000),
                                            (27, 96, 96, 20000), (27, 256, 256, 6000), (27, 128, 96, 20000),
                                            (8, 64, 128, 30000), (27, 32, 64, 300)])
def test_wgrad_tcgen05_matches_explicit_formulas(dtype, K, c_in, c_out, n):
    """dW on the tensor cores (operands read as MN-major tiles, units of 64 or 32 channels grouped on
    the M side, fp32 accumulation, split over row ranges) against a per-offset fp32 GEMM on the same
    quantised operands."""
    from warpconvnet_b200.nn.functional.sparse_conv import sparse_conv_wgrad
    coords, _, _ = _layer_case(n, 4, 4, 91, "raster_crop")
    coords = np.ascontiguousarray(coords[np.argsort(km.morton_code(coords[:, 1:]), kind="stable")])
    c = torch.from_numpy(coords).to(DEV)
    g = torch.Generator().manual_seed(K * c_in + c_out)
    if K == 27:
        kmap, n_out = generate_kernel_map(c, c, (1, 1, 1), (3, 3, 3)), n
        i, o, f, _ = km.generate_kernel_map(coords, coords, (1, 1, 1), (3, 3, 3))
    else:
        coarse, _ = stride_coords(c, (2, 2, 2))
        kmap, n_out = generate_kernel_map(c, coarse, (2, 2, 2), (2, 2, 2)), len(coarse)
        i, o, f, _ = km.generate_kernel_map(coords, coarse.cpu().numpy(), (2, 2, 2), (2, 2, 2))
    x = torch.randn(n, c_in, generator=g).to(dtype)
    go = torch.randn(n_out, c_out, generator=g).to(dtype)
    gw = sparse_conv_wgrad(x.to(DEV), go.to(DEV), kmap, n_out)
    check_device_status(DEV)
    assert gw is not None and gw.dtype == torch.float32 and tuple(gw.shape) == (K, c_in, c_out)
    ref = torch.zeros(K, c_in, c_out)
    for k in range(K):
        s, e = int(f[k]), int(f[k + 1])
        if e > s:
            ref[k] = x.float()[torch.from_numpy(i[s:e]).long()].T @ go.float()[torch.from_numpy(o[s:e]).long()]
    assert rel_l2(gw.cpu().numpy(), ref.numpy()) < 1e-4  # fp32 accumulation of exact products
    # the same through the tiled table (dY rows read through the row order)
    gt = sparse_conv_wgrad(x.to(DEV), go.to(DEV), kmap, n_out, tile_order=True)
    check_device_status(DEV)
    assert rel_l2(gt.cpu().numpy(), ref.numpy()) < 1e-4


def test_backward_native_dx_strided_and_transposed_fp16():
    """dX of a stride-2 convolution and of its transposed counterpart through the forward kernel on
    the swapped table (tensor-core path, fp16) against autograd over the explicit formulas in fp32."""
    from warpconvnet_b200 import SPARSE_CONV_BWD_ALGO_MODE as BWD
    n, c_in, c_out = 20000, 32, 64
    coords, x, _ = _layer_case(n, c_in, c_out, 21, "raster_crop")
    g = torch.Generator().manual_seed(4)
    w = torch.randn(8, c_in, c_out, generator=g) * 0.1
    xq, wq = x.half(), w.half()
    xg = xq.clone().to(DEV).requires_grad_(True)
    vox = make_voxels(coords, xg)
    down = spatially_sparse_conv(vox, wq.to(DEV), 2, stride=2, fwd_algo=ALGO.IMPLICIT_GEMM, bwd_algo=BWD.IMPLICIT_GEMM)
    go = torch.randn(down.feature_tensor.shape, generator=g).half()
    down.feature_tensor.backward(go.to(DEV))
    # reference: the same map from the oracle, explicit formulas in fp32
    out_c, _ = km.stride_coords(coords, (2, 2, 2))
    i, o, f, _ = km.generate_kernel_map(coords, out_c, (2, 2, 2), (2, 2, 2))
    # the product's strided rows are in first-occurrence order, as the oracle's: same row numbering
    ref = torch.zeros(n, c_in)
    for k in range(8):
        s, e = int(f[k]), int(f[k + 1])
        ref.index_add_(0, torch.from_numpy(i[s:e]).long(), go.float()[torch.from_numpy(o[s:e]).long()] @ wq.float()[k].T)
    assert rel_l2(xg.grad.float().cpu().numpy(), ref.numpy()) < 1e-2
    # transposed convolution back up: its dX reads the forward (down) table
    wt = (torch.randn(8, c_out, c_in, generator=g) * 0.1).half()
    cg = down.feature_tensor.detach().clone().requires_grad_(True)
    up = spatially_sparse_conv(down.replace(batched_features=cg), wt.to(DEV), 2, stride=2, transposed=True,
                               output_spatially_sparse_tensor=vox, fwd_algo=ALGO.IMPLICIT_GEMM,
                               bwd_algo=BWD.IMPLICIT_GEMM)
    gu = torch.randn(n, c_in, generator=g).half()
    up.feature_tensor.backward(gu.to(DEV))
    ref2 = torch.zeros(len(out_c), c_out)
    for k in range(8):  # up[i] += coarse[o] @ wt[k]  =>  d coarse[o] += d up[i] @ wt[k]^T
        s, e = int(f[k]), int(f[k + 1])
        ref2.index_add_(0, torch.from_numpy(o[s:e]).long(), gu.float()[torch.from_numpy(i[s:e]).long()] @ wt.float()[k].T)
    assert rel_l2(cg.grad.float().cpu().numpy(), ref2.numpy()) < 1e-2
    check_device_status(DEV)


def test_surface_errors_and_shortcuts():
    n = 2000
    coords, x, w = _layer_case(n, 8, 12, 5, "sample")
    vox = make_voxels(coords, x)
    with pytest.raises(TypeError):
        spatially_sparse_conv(x.to(DEV), w.to(DEV), 3)
    with pytest.raises(AssertionError):
        spatially_sparse_conv(vox, w[:8].to(DEV), 2, stride=2, transposed=True)
    with pytest.raises(ValueError):
        spatially_sparse_conv(vox, w.to(DEV), 3, fwd_algo="winograd")
    # 1x1x1: a plain matmul, coordinates and cache untouched
    w1 = torch.randn(1, 8, 5)
    b = torch.randn(5)
    y = spatially_sparse_conv(vox, w1.to(DEV), 1, bias=b.to(DEV))
    assert rel_l2(y.feature_tensor.cpu().numpy(), (x @ w1[0] + b).numpy()) < 1e-5 and vox.cache is None
    # list of algorithms, string algorithm, bias on the fused path
    y2 = spatially_sparse_conv(vox, w.to(DEV), 3, bias=torch.ones(12, device=DEV),
                               fwd_algo=[ALGO.EXPLICIT_GEMM, ALGO.IMPLICIT_GEMM])
    y3 = spatially_sparse_conv(vox, w.to(DEV), 3, bias=torch.ones(12, device=DEV), fwd_algo="explicit_gemm")
    assert rel_l2(y2.feature_tensor.cpu().numpy(), y3.feature_tensor.cpu().numpy()) < 1e-5
    # a compact user-supplied map drives the fused kernel too
    i, o, f, iden = km.generate_kernel_map(coords, coords, (1, 1, 1), (3, 3, 3))
    user = IntSearchResult(torch.from_numpy(i).to(DEV), torch.from_numpy(o).to(DEV), torch.from_numpy(f), iden)
    y4 = sparse_conv_fused(x.to(DEV), w.to(DEV), user, n)
    assert rel_l2(y4.cpu().numpy(), (y3.feature_tensor - 1).cpu().numpy()) < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_minkunet_matches_oracle(dtype):
    """U-Net forward (all layer kinds: 1x1, 3x3x3, stride-2 down, transposed up, skip concat,
    fused BN/ReLU/residual) against the CPU restatement of the reference model."""
    scenes = [synthetic.room_scene(6000, 0.05, 600 + s, "raster_crop") for s in range(2)]
    coords, offsets = synthetic.batch_scenes(scenes)
    feats = torch.rand(len(coords), 3, generator=torch.Generator().manual_seed(0))
    torch.manual_seed(0)
    model = MinkUNet18(3, 20)
    randomize_batchnorm_(model, 1)
    model.eval()
    ref = osc.minkunet_forward(model.state_dict(), coords, feats, layers=(2,) * 8).numpy()
    m = model.to(DEV).to(dtype)
    vox = Voxels(torch.from_numpy(coords[:, 1:].copy()).to(DEV), feats.to(DEV).to(dtype), offsets=torch.from_numpy(offsets))
    with torch.no_grad():
        out = m(vox)
    check_device_status(DEV)
    assert out.feature_tensor.shape == (len(coords), 20)
    err = rel_l2(out.feature_tensor.float().cpu().numpy(), ref)
    assert err < (1e-4 if dtype == torch.float32 else 2e-2), err
    # 5 3x3x3 maps + 4 down maps + the transposed views the output-side kernel needed (a layer run from the
    # input side reads the down map itself)
    assert len(out.cache) == 13 if dtype == torch.float32 else 9 <= len(out.cache) <= 13
