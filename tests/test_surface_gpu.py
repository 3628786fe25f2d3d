"""The reference's user-facing surface beyond the convolution itself: ``Voxels`` construction and
conversions, Morton ordering per batch segment, the ``order=`` argument of the convolution, 2-D
convolution, custom kernel centres.  Bodies follow the reference's own tests
(tests/types/test_voxels.py, tests/coords/test_serialization.py)."""
import numpy as np
import pytest
import torch

from oracle import kernel_map as km
from oracle import sparse_conv as osc
from warpconvnet_b200 import (POINT_ORDERING, SPARSE_CONV_FWD_ALGO_MODE as ALGO, SparseConv2d, SparseConv3d, Voxels,
                              generate_kernel_map, spatially_sparse_conv)
from warpconvnet_b200._native import check_device_status
from warpconvnet_b200.geometry.coords.ops.batch_index import batch_indexed_coordinates
from warpconvnet_b200.geometry.coords.ops.serialization import encode, morton_code

from conftest import rel_l2

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


@pytest.fixture(scope="module")
def voxels_and_sizes():
    """Three clouds of random cells with repeats, as lists of per-item tensors (test_voxels.py:16-27)."""
    g = torch.Generator().manual_seed(0)
    sizes = torch.randint(20000, 60000, (3,), generator=g)
    coords = [(torch.rand((int(n), 3), generator=g) / 0.01).int() for n in sizes]
    feats = [torch.rand((int(n), 7), generator=g) for n in sizes]
    return Voxels(coords, feats), sizes


def test_voxels_from_lists_and_device_move(voxels_and_sizes):
    vox, sizes = voxels_and_sizes
    ends = sizes.cumsum(0).tolist()
    assert vox.batched_coordinates.batch_size == 3 and vox.batched_features.batch_size == 3
    assert vox.batched_coordinates.offsets.tolist() == [0] + ends
    assert tuple(vox.batched_coordinates.batched_tensor.shape) == (ends[-1], 3)
    assert tuple(vox.batched_features.batched_tensor.shape) == (ends[-1], 7)
    assert vox.batch_size == 3 and vox.num_channels == 7 and len(vox) == ends[-1]
    on_gpu = vox.to(DEV)
    assert on_gpu.batched_coordinates.batched_tensor.device == DEV and on_gpu.feature_tensor.device == DEV
    item = on_gpu[1]  # one batch item as a batch of one
    assert len(item) == int(sizes[1]) and item.offsets.tolist() == [0, int(sizes[1])]
    assert torch.equal(item.coordinate_tensor, on_gpu.coordinate_tensor[ends[0]:ends[1]])


def test_voxels_unique_counts_distinct_rows(voxels_and_sizes):
    vox = voxels_and_sizes[0].to(DEV)
    uniq = vox.unique()
    bc = batch_indexed_coordinates(vox.batched_coordinates.batched_tensor, vox.offsets)
    distinct = torch.unique(bc, dim=0)
    assert len(uniq.batched_coordinates) == distinct.shape[0] < len(vox)
    assert torch.equal(torch.unique(uniq.batch_indexed_coordinates, dim=0), distinct)
    # the surviving feature rows belong to their coordinates (first occurrence wins)
    first = {}
    for r, row in enumerate(bc[:2000].tolist()):
        first.setdefault(tuple(row), r)
    got = {tuple(c): f for c, f in zip(uniq.batch_indexed_coordinates[:200].tolist(), uniq.feature_tensor[:200])}
    for key, f in list(got.items())[:50]:
        if key in first:
            assert torch.equal(f, vox.feature_tensor[first[key]])
    check_device_status(DEV)


@pytest.mark.parametrize("in_dtype,amp_dtype", [(torch.float32, torch.float16), (torch.float32, torch.bfloat16),
                                                (torch.float16, torch.float16), (torch.float16, torch.bfloat16)])
def test_voxels_feature_tensor_follows_autocast(voxels_and_sizes, in_dtype, amp_dtype):
    vox = voxels_and_sizes[0].to(DEV).to(dtype=in_dtype)
    with torch.autocast("cuda", dtype=amp_dtype):
        f = vox.features
        assert f.dtype == amp_dtype
        assert vox.batched_features.batched_tensor.dtype == in_dtype
        assert (f + 1.0).dtype == f.dtype
    assert vox.features.dtype == in_dtype


@pytest.mark.parametrize("in_dtype,out_dtype", [(torch.float32, torch.float16), (torch.float32, torch.bfloat16),
                                                (torch.float16, torch.float32), (torch.bfloat16, torch.float32)])
def test_voxels_dtype_conversion(voxels_and_sizes, in_dtype, out_dtype):
    vox = voxels_and_sizes[0].to(DEV, dtype=in_dtype)
    conv = vox.to(dtype=out_dtype)
    assert conv.features.dtype == out_dtype and vox.features.dtype == in_dtype
    assert (conv + 1.0).features.dtype == out_dtype
    assert conv.coordinate_tensor.dtype == vox.coordinate_tensor.dtype


def test_extra_attributes_survive_replace():
    g = torch.Generator().manual_seed(3)
    coords = [torch.floor(torch.rand((n, 3), generator=g) / 0.01).int() for n in (1500, 900, 4000)]
    feats = [torch.rand((len(c), 7), generator=g) for c in coords]
    vox = Voxels(coords, feats, device="cuda:0", test_attribute="test", voxel_size=0.01)
    rep = vox.replace(batched_features=vox.batched_features + 1)
    assert rep.extra_attributes["test_attribute"] == "test" and rep.voxel_size == 0.01
    assert torch.equal(rep.feature_tensor, vox.feature_tensor + 1)
    assert rep.cache is vox.cache


def test_encode_orders_every_batch_segment(voxels_and_sizes):
    """``encode(..., batch_offsets, return_perm=True)``: the permutation keeps every row inside its
    batch segment and sorts the segment by Morton code (test_serialization.py:89-114)."""
    vox = voxels_and_sizes[0].to(DEV)
    coords, offsets = vox.coordinate_tensor, vox.offsets
    codes = morton_code(coords)
    assert codes.dtype == torch.int64 and np.array_equal(codes.cpu().numpy(), km.morton_code(coords.cpu().numpy()))
    res = encode(coords, batch_offsets=offsets, order=POINT_ORDERING.MORTON_XYZ, return_perm=True, return_inverse=True)
    perm = res.perm
    assert perm.dtype == torch.int64 and torch.equal(torch.sort(perm).values, torch.arange(len(perm), device=DEV))
    for b in range(len(offsets) - 1):
        s, e = int(offsets[b]), int(offsets[b + 1])
        seg = perm[s:e]
        assert int(seg.min()) >= s and int(seg.max()) < e
        sorted_codes = codes[seg]
        assert bool((sorted_codes[1:] >= sorted_codes[:-1]).all())
    assert torch.equal(res.inverse_perm[perm], torch.arange(len(perm), device=DEV))
    # Voxels.sort takes its codes from the minimum rounded down to a multiple of 16: the same kind of
    # order (per-segment, non-decreasing in its own codes, a permutation of the rows)
    sorted_vox = vox.sort(POINT_ORDERING.MORTON_XYZ)
    origin = sorted_vox.batched_coordinates.morton_origin
    assert origin is not None and bool((origin % 16 == 0).all()) and bool((origin <= coords.min(0).values).all())
    sperm, scode = sorted_vox.extra_attributes["perm"], sorted_vox.extra_attributes["code"]
    assert torch.equal(sorted_vox.coordinate_tensor, coords[sperm]) and sorted_vox.ordering == POINT_ORDERING.MORTON_XYZ
    assert torch.equal(scode, morton_code(coords, origin=origin))
    for b in range(len(offsets) - 1):
        s, e = int(offsets[b]), int(offsets[b + 1])
        seg = scode[sperm[s:e]]
        assert int(sperm[s:e].min()) >= s and int(sperm[s:e].max()) < e and bool((seg[1:] >= seg[:-1]).all())
    assert sorted_vox.sort(POINT_ORDERING.MORTON_XYZ) is sorted_vox


@pytest.mark.parametrize("order", [POINT_ORDERING.MORTON_XYZ, POINT_ORDERING.MORTON_ZYX])
def test_conv_order_argument_sorts_the_output_rows(order):
    """``order=`` on a strided convolution (sparse_conv.py:1889-1897 of the reference): the output
    coordinates come Morton-sorted per batch item and the features are those of the unordered call,
    row for row."""
    rng = np.random.default_rng(12)
    xyz = [np.unique(rng.integers(0, 40, size=(n, 3)).astype(np.int32), axis=0) for n in (5000, 3000)]
    coords = [torch.from_numpy(c) for c in xyz]
    g = torch.Generator().manual_seed(1)
    feats = [torch.randn(len(c), 16, generator=g) for c in coords]
    vox = Voxels(coords, feats).to(DEV)
    w = (torch.randn(8, 16, 24, generator=g) * 0.2).to(DEV)
    with torch.no_grad():
        plain = spatially_sparse_conv(vox, w, 2, stride=2, fwd_algo=ALGO.IMPLICIT_GEMM)
        vox2 = Voxels(coords, feats).to(DEV)  # fresh cache: the ordered call builds its own map
        ordered = spatially_sparse_conv(vox2, w, 2, stride=2, fwd_algo=ALGO.IMPLICIT_GEMM, order=order)
    oc = ordered.batch_indexed_coordinates
    assert ordered.offsets.tolist() == plain.offsets.tolist() and ordered.tensor_stride == (2, 2, 2)
    all_codes = morton_code(oc[:, 1:], order=order)  # one origin for the whole batch, as encode uses
    for b in range(2):
        s, e = int(ordered.offsets[b]), int(ordered.offsets[b + 1])
        assert bool((oc[s:e, 0] == b).all())
        codes = all_codes[s:e]
        assert bool((codes[1:] >= codes[:-1]).all())
    # same rows, other order: match them up through a hash of the coordinates
    def keyed(v):
        c = v.batch_indexed_coordinates.cpu().numpy().astype(np.int64)
        key = ((c[:, 0] * 64 + c[:, 1]) * 64 + c[:, 2]) * 64 + c[:, 3]
        idx = np.argsort(key)
        return key[idx], v.feature_tensor.cpu().numpy()[idx]
    ka, fa = keyed(plain)
    kb, fb = keyed(ordered)
    assert np.array_equal(ka, kb) and np.array_equal(fa, fb)
    check_device_status(DEV)


def test_sparse_conv2d_matches_oracle():
    """Two spatial dimensions: a 3x3 window, a strided 2x2 window and its transposed counterpart
    against the oracle run on the z = 0 slab (a kx x ky window is a kx x ky x 1 window there)."""
    rng = np.random.default_rng(21)
    xy = [np.unique(rng.integers(-30, 30, size=(n, 2)).astype(np.int32), axis=0) for n in (2500, 1200)]
    g = torch.Generator().manual_seed(2)
    feats = [torch.randn(len(c), 8, generator=g) for c in xy]
    vox = Voxels([torch.from_numpy(c) for c in xy], feats).to(DEV)
    assert vox.num_spatial_dims == 2
    torch.manual_seed(0)
    conv = SparseConv2d(8, 12, 3, bias=True).to(DEV)
    down = SparseConv2d(12, 12, 2, stride=2, bias=False).to(DEV)
    up = SparseConv2d(12, 8, 2, stride=2, bias=False, transposed=True).to(DEV)
    assert tuple(conv.weight.shape) == (9, 8, 12)
    with torch.no_grad():
        a = conv(vox)
        b = down(a)
        c = up(b, vox)
    check_device_status(DEV)
    slab = np.concatenate([np.concatenate([np.full((len(c_), 1), i, np.int32), c_, np.zeros((len(c_), 1), np.int32)], 1)
                           for i, c_ in enumerate(xy)], 0)
    x = torch.cat(feats)
    i, o, f, iden = km.generate_kernel_map(slab, slab, (1, 1, 1), (3, 3, 1))
    ya = osc.explicit_gemm_forward(x, conv.weight.detach().cpu(), i, o, f, iden, len(slab)) + conv.bias.detach().cpu()
    assert rel_l2(a.feature_tensor.cpu().numpy(), ya.numpy()) < 1e-4
    coarse, coarse_off = km.stride_coords(slab, (2, 2, 1))
    assert np.array_equal(b.batch_indexed_coordinates.cpu().numpy(), coarse[:, :3]) and b.tensor_stride == (2, 2)
    i2, o2, f2, _ = km.generate_kernel_map(slab, coarse, (2, 2, 1), (2, 2, 1))
    yb = osc.explicit_gemm_forward(ya, down.weight.detach().cpu(), i2, o2, f2, None, len(coarse))
    assert rel_l2(b.feature_tensor.cpu().numpy(), yb.numpy()) < 1e-4
    ti, to, tf, _ = km.transposed_kernel_map(coarse, slab, (2, 2, 1), (2, 2, 1))
    yc = osc.explicit_gemm_forward(yb, up.weight.detach().cpu(), ti, to, tf, None, len(slab))
    assert len(c) == len(vox) and c.tensor_stride == (1, 1)
    assert rel_l2(c.feature_tensor.cpu().numpy(), yc.numpy()) < 1e-4


def test_custom_kernel_center_matches_reference_fixture(golden):
    """method="offset" with a window centre of the caller's choice, against the table the
    reference's offset-list kernel produced for the same window (tests/golden/kmap_extra.npz)."""
    g = golden("kmap_extra.npz")
    c = torch.from_numpy(g["coords"]).to(DEV)
    res = generate_kernel_map(c, c, (1, 1, 1), (3, 2, 3), kernel_center_offset=tuple(int(v) for v in g["center"]),
                              method="offset")
    assert np.array_equal(res.neighbor_table(len(g["coords"])).cpu().numpy(), g["found_c"])
    assert res.identity_map_index is None
    with pytest.raises(AssertionError):
        generate_kernel_map(c, c, (1, 1, 1), (3, 2, 3), kernel_center_offset=(0, 1, 2), method="size")
    dil = generate_kernel_map(c, c, (1, 1, 1), (3, 3, 3), kernel_dilation=tuple(int(v) for v in g["dilation"]),
                              method="offset")
    assert np.array_equal(dil.neighbor_table(len(g["coords"])).cpu().numpy(), g["found_d"])
    coarse = torch.from_numpy(g["coarse"]).to(DEV)
    dils = generate_kernel_map(c, coarse, (2, 2, 2), (3, 3, 3), kernel_dilation=tuple(int(v) for v in g["dilation"]))
    assert np.array_equal(dils.neighbor_table(len(g["coarse"])).cpu().numpy(), g["found_ds"])
    check_device_status(DEV)
