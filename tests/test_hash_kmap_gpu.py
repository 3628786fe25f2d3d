"""GPU parity: hash table, kernel map, strided coordinates and Morton code against
the oracle and the golden vectors generated from the reference (bit-exact)."""
import numpy as np
import pytest
import torch

from oracle import kernel_map as km
from warpconvnet_b200 import (HashMethod, IntSearchResult, TorchHashTable, generate_kernel_map, morton_code,
                              stride_coords)
from warpconvnet_b200._native import check_device_status
from warpconvnet_b200.datasets import synthetic
from warpconvnet_b200.geometry.coords.ops.stride import unique_strided_rows
from warpconvnet_b200.geometry.coords.search.torch_discrete import _kernel_map_from_size

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def assert_map_equal(res: IntSearchResult, i, o, f):
    assert np.array_equal(res.offsets.numpy(), f)
    assert np.array_equal(res.in_maps.cpu().numpy(), i)
    assert np.array_equal(res.out_maps.cpu().numpy(), o)


@pytest.mark.parametrize("method", list(HashMethod))
def test_hash_search_golden(golden, method):
    g = golden("kmap_small.npz")
    t = TorchHashTable.from_keys(dev(g["coords"]), hash_method=method)
    assert t.capacity == max(16, 2 * len(g["coords"])) and t.key_dim == 4
    r = t.search(dev(g["queries"])).cpu().numpy()
    assert np.array_equal(r, g["search"])
    # every inserted key is found at its own row; absent keys give -1
    assert np.array_equal(t.search(dev(g["coords"])).cpu().numpy(), np.arange(len(g["coords"]), dtype=np.int32))
    check_device_status(DEV)


def test_hash_duplicates_and_unique_index():
    rng = np.random.default_rng(5)
    base = rng.integers(0, 6, size=(5000, 4)).astype(np.int32)
    t = TorchHashTable(2 * len(base))
    t.insert(dev(base))
    r = t.search(dev(base)).cpu().numpy()
    assert np.array_equal(r, km.hash_search(base, base))  # smallest row index of each key
    uniq = t.unique_index.cpu().numpy()
    assert len(uniq) == len(np.unique(base, axis=0))
    assert np.array_equal(np.unique(base[uniq], axis=0), np.unique(base, axis=0))
    d = t.to_dict()
    t2 = TorchHashTable.from_dict(d, device=DEV)
    assert np.array_equal(t2.search(dev(base)).cpu().numpy(), r)


def test_hash_errors():
    t = TorchHashTable(16)
    with pytest.raises(RuntimeError):
        t.search(torch.zeros(1, 4, dtype=torch.int32, device=DEV))
    with pytest.raises(AssertionError):
        t.insert(torch.zeros(9, 4, dtype=torch.int32, device=DEV))  # > capacity / 2
    with pytest.raises(ValueError):
        t.insert(torch.zeros(4, dtype=torch.int32, device=DEV))
    with pytest.raises(TypeError):
        t.insert(torch.zeros(2, 4, dtype=torch.float32, device=DEV))
    with pytest.raises(ValueError):
        t.insert(torch.zeros(2, 4, dtype=torch.int32))


@pytest.mark.parametrize("tag,stride,ks", [("333", (1, 1, 1), (3, 3, 3)), ("222", (2, 2, 2), (2, 2, 2)),
                                            ("312", (1, 1, 1), (3, 1, 2))])
def test_kernel_map_golden(golden, tag, stride, ks):
    g = golden("kmap_small.npz")
    out_coords = g["out_coords"] if tag == "222" else g["coords"]
    res = generate_kernel_map(dev(g["coords"]), dev(out_coords), stride, ks)
    assert res.identity_map_index == (13 if tag == "333" else None)
    nbr = res.neighbor_table(len(out_coords)).cpu().numpy()
    assert np.array_equal(nbr, km.kernel_map_found(g["coords"], out_coords, stride, ks))
    assert_map_equal(res, g["in" + tag], g["out" + tag], g["off" + tag])
    # per-offset slices and the dense form rebuilt from the compact one
    a, b = res[5]
    assert len(a) == res.numel(5) == int(g["off" + tag][6] - g["off" + tag][5])
    rebuilt = IntSearchResult(res.in_maps, res.out_maps, res.offsets).neighbor_table(len(out_coords))
    assert np.array_equal(rebuilt.cpu().numpy(), nbr)


def test_transposed_map_golden(golden):
    g = golden("kmap_small.npz")
    fwd = generate_kernel_map(dev(g["coords"]), dev(g["out_coords"]), (2, 2, 2), (2, 2, 2))
    tr = fwd.swapped(num_in=len(g["coords"]))
    nbr_t = tr.neighbor_table(len(g["coords"])).cpu().numpy()
    expect = np.full((8, len(g["coords"])), -1, np.int32)
    for k in range(8):
        s, e = g["tr_off"][k], g["tr_off"][k + 1]
        expect[k, g["tr_out"][s:e]] = g["tr_in"][s:e]
    assert np.array_equal(nbr_t, expect)
    assert_map_equal(tr, g["tr_in"], g["tr_out"], g["tr_off"])


@pytest.mark.parametrize("method", list(HashMethod))
def test_kernel_map_vs_direct_search(method):
    """Per-offset map equals a direct hash search of out*stride + offset
    (the check of the reference's tests/nn/test_sparse_conv.py:109-134)."""
    scenes = [synthetic.room_scene(20000, 0.05, 310 + s, "sample") for s in range(2)]
    coords, _ = synthetic.batch_scenes(scenes)
    c = dev(coords)
    res = generate_kernel_map(c, c, (1, 1, 1), (3, 3, 3), hash_method=method)
    table = TorchHashTable.from_keys(c, hash_method=method)
    offs = km.kernel_offsets_from_size((3, 3, 3))
    for k in (0, 7, 13, 26):
        direct = table.search(c + dev(offs[k])[None, :]).cpu().numpy()
        i, o = res[k]
        hit = direct >= 0
        assert np.array_equal(i.cpu().numpy(), direct[hit]) and np.array_equal(o.cpu().numpy(), np.nonzero(hit)[0])
    a = km.generate_kernel_map(coords, coords, (1, 1, 1), (3, 3, 3))
    assert_map_equal(res, *a[:3])


def test_skip_symmetric_is_prefix():
    """skip_symmetric map = first K//2 offsets of the full map (tests/nn/test_sparse_conv.py:137-181)."""
    xyz = synthetic.random_cells(5000, 24, seed=2)
    c = dev(np.concatenate([np.zeros((len(xyz), 1), np.int32), xyz], 1))
    full = generate_kernel_map(c, c, (1, 1, 1), (3, 3, 3))
    half = generate_kernel_map(c, c, (1, 1, 1), (3, 3, 3), skip_symmetric_kernel_map=True)
    assert len(half) == 13 and half.identity_map_index == 13
    n = int(full.offsets[13])
    assert np.array_equal(half.offsets.numpy(), full.offsets.numpy()[:14])
    assert torch.equal(half.in_maps, full.in_maps[:n]) and torch.equal(half.out_maps, full.out_maps[:n])


def test_kernel_map_edge_cases():
    # single voxel
    one = torch.tensor([[0, 5, -3, 2]], dtype=torch.int32, device=DEV)
    res = generate_kernel_map(one, one, (1, 1, 1), (3, 3, 3))
    assert res.offsets.tolist() == [0] * 14 + [1] * 14
    assert res.in_maps.tolist() == [0] and res.out_maps.tolist() == [0]
    # no query at all
    empty = torch.zeros((0, 4), dtype=torch.int32, device=DEV)
    res = generate_kernel_map(one, empty, (1, 1, 1), (3, 3, 3))
    assert res.offsets.tolist() == [0] * 28 and len(res.in_maps) == 0
    # a batch item without voxels, coordinates near the int range
    c = np.array([[0, 2**30, -2**30, 7], [0, 2**30 + 1, -2**30, 7], [2, 0, 0, 0], [2, 0, 0, 1]], np.int32)
    res = generate_kernel_map(dev(c), dev(c), (1, 1, 1), (3, 3, 3))
    exp = km.generate_kernel_map(c, c, (1, 1, 1), (3, 3, 3))
    assert_map_equal(res, *exp[:3])
    with pytest.raises(AssertionError):
        generate_kernel_map(dev(c).long(), dev(c), (1, 1, 1), (3, 3, 3))
    with pytest.raises(AssertionError):
        generate_kernel_map(dev(c), dev(c), (1, 1, 1), (3, 3, 3), kernel_center_offset=(0, 0, 0))


def test_stride_coords(golden):
    g = golden("kmap_small.npz")
    out, offsets = stride_coords(dev(g["coords"]), (2, 2, 2))
    assert np.array_equal(out.cpu().numpy(), g["out_coords"])  # first-occurrence order, as the oracle
    assert offsets.tolist() == np.concatenate([[0], np.cumsum(np.bincount(g["out_coords"][:, 0]))]).tolist()
    rows, uidx, parent = unique_strided_rows(dev(g["coords"]), (2, 2, 2), return_parent=True)
    q = np.floor_divide(g["coords"], np.array([1, 2, 2, 2]))
    assert np.array_equal(rows.cpu().numpy()[parent.cpu().numpy()], q)
    assert np.array_equal(q[uidx.cpu().numpy()], rows.cpu().numpy()) and (np.diff(uidx.cpu().numpy()) > 0).all()
    same, offs1 = stride_coords(dev(g["coords"]), (1, 1, 1))
    assert same.shape[0] == len(g["coords"]) and offs1[-1] == len(g["coords"])
    # anisotropic stride with negatives: floor division, not truncation
    out2, _ = stride_coords(dev(g["coords"]), (2, 1, 3))
    exp2, _ = km.stride_coords(g["coords"], (2, 1, 3))
    assert np.array_equal(out2.cpu().numpy(), exp2)


def test_morton(golden):
    g = golden("kmap_small.npz")
    xyz = dev(g["morton_xyz"].astype(np.int32))
    codes = morton_code(xyz)
    assert np.array_equal(codes.cpu().numpy(), g["morton"])
    shifted = morton_code(xyz - 1000)  # the minimum is subtracted first
    assert torch.equal(shifted, codes)
    big = torch.tensor([[0, 0, 0], [2**20 - 1, 2**20 - 1, 2**20 - 1], [1, 0, 0], [0, 1, 0], [0, 0, 1]],
                       dtype=torch.int32, device=DEV)
    assert morton_code(big).tolist() == [0, 2**60 - 1, 1, 2, 4]


@pytest.mark.parametrize("mode,n_per_scene", [("raster_crop", 250000), ("sample", 250000)])
def test_kernel_map_full_size_properties(mode, n_per_scene):
    """Config-2 size (4 rooms x 250k voxels): properties that need no CPU replay —
    symmetry of the 3x3x3 map, one parent per voxel in the 2x2x2 map, swap involution —
    plus a replay of a slice against the oracle."""
    scenes = [synthetic.room_scene(n_per_scene, 0.02, 100 + s, mode) for s in range(4)]
    coords, _ = synthetic.batch_scenes(scenes)
    c = dev(coords)
    res = generate_kernel_map(c, c, (1, 1, 1), (3, 3, 3))
    nbr = res.neighbor_table(len(coords))
    n = len(coords)
    ar = torch.arange(n, device=DEV, dtype=torch.int32)
    assert torch.equal(nbr[13], ar)
    for k in (0, 4, 12):  # pair (m -> j at k) <=> (j -> m at 26-k)
        j = nbr[k].long()
        hit = j >= 0
        assert torch.equal(nbr[26 - k][j[hit]], ar[hit])
    off = res.offsets
    assert off[-1] == int((nbr >= 0).sum()) and all(int(off[k + 1] - off[k]) == int(off[27 - k] - off[26 - k]) for k in range(13))
    sub = slice(0, 3000)
    exp = km.kernel_map_found(coords, coords[sub], (1, 1, 1), (3, 3, 3))
    assert np.array_equal(nbr[:, sub].cpu().numpy(), exp)
    out, offsets = stride_coords(c, (2, 2, 2))
    exp_out, _ = km.stride_coords(coords, (2, 2, 2))
    assert np.array_equal(out.cpu().numpy(), exp_out)
    down = generate_kernel_map(c, out, (2, 2, 2), (2, 2, 2))
    assert int(down.offsets[-1]) == n and len(torch.unique(down.in_maps)) == n
    up = down.swapped(num_in=n)
    assert int((up.neighbor_table(n) >= 0).sum(0).min()) == 1 and int((up.neighbor_table(n) >= 0).sum(0).max()) == 1
    check_device_status(DEV)


@pytest.mark.parametrize("n,ksize,stride", [(30000, (3, 3, 3), (1, 1, 1)), (4096, (3, 3, 3), (1, 1, 1)),
                                             (5000, (2, 2, 2), (2, 2, 2)), (37, (3, 3, 3), (1, 1, 1)),
                                             (70000, (3, 3, 3), (1, 1, 1)), (20000, (3, 1, 3), (1, 1, 1))])
def test_tile_order_matches_oracle(n, ksize, stride):
    """Tiled neighbour table: rows of each window (4096 rows for small tables, 16384 otherwise) sorted by
    the presence key (3x3x3: rare offsets in the high bits), ties by row; bit-exact against the oracle's
    restatement, for a forward and a transposed (one-hot) map, several windows and a ragged last one."""
    coords = synthetic.room_scene(n, 0.02, 41, "raster_crop")
    coords = np.concatenate([np.zeros((len(coords), 1), np.int32), coords], axis=1).astype(np.int32)
    coords = np.ascontiguousarray(coords[np.argsort(km.morton_code(coords[:, 1:]), kind="stable")])
    if stride == (1, 1, 1):
        out = coords
    else:
        out, _ = km.stride_coords(coords, stride)
    res = generate_kernel_map(dev(coords), dev(out), stride, ksize)
    cases = [(res, len(out))]
    if stride != (1, 1, 1):
        cases.append((res.swapped(num_in=len(coords)), len(coords)))
    for r, m in cases:
        nbr = r.neighbor_table(m).cpu().numpy()
        tiled, rows = r.tiled_neighbor_table(m)
        want_rows, want_tiled = km.tile_order(nbr)
        assert np.array_equal(rows.cpu().numpy(), want_rows)
        assert np.array_equal(tiled.cpu().numpy(), want_tiled)
        assert np.array_equal(np.sort(want_rows), np.arange(m))
        w = km.tile_order_window(m)
        assert np.array_equal(want_rows // w, np.arange(m) // w)  # no row leaves its window
    check_device_status(DEV)


@pytest.mark.parametrize("method", list(HashMethod))
def test_self_map_with_repeated_rows_matches_oracle(method):
    """A coordinate set searched against itself takes the mirrored search when its rows are
    distinct and the full search when they are not (the table records which); both equal the
    oracle, compact form included."""
    rng = np.random.default_rng(17)
    distinct = np.unique(rng.integers(0, 24, size=(6000, 4)).astype(np.int32), axis=0)
    distinct[:, 0] %= 2
    distinct = np.unique(distinct, axis=0)
    rng.shuffle(distinct)
    repeated = np.concatenate([distinct, distinct[:500]], axis=0)
    for coords in (distinct, repeated):
        c = dev(coords)
        res = generate_kernel_map(c, c, (1, 1, 1), (3, 3, 3), hash_method=method)
        i, o, f, iden = km.generate_kernel_map(coords, coords, (1, 1, 1), (3, 3, 3))
        assert np.array_equal(res.neighbor_table(len(coords)).cpu().numpy(),
                              km.kernel_map_found(coords, coords, (1, 1, 1), (3, 3, 3)))
        assert_map_equal(res, i, o, f)
    # a 3x1x5 window: mirrored offsets with unequal extents
    c = dev(distinct)
    res = generate_kernel_map(c, c, (1, 1, 1), (3, 1, 5), hash_method=method)
    assert np.array_equal(res.neighbor_table(len(distinct)).cpu().numpy(),
                          km.kernel_map_found(distinct, distinct, (1, 1, 1), (3, 1, 5)))
    check_device_status(DEV)


@pytest.mark.parametrize("dilation", [(2, 2, 2), (1, 3, 2)])
def test_dilated_kernel_maps_match_oracle(dilation):
    """Dilated windows: the self map (mirrored search) and a strided map against the oracle."""
    rng = np.random.default_rng(23)
    coords = np.unique(rng.integers(-9, 9, size=(5000, 4)).astype(np.int32), axis=0)
    coords[:, 0] = np.abs(coords[:, 0]) % 2
    coords = np.unique(coords, axis=0)
    rng.shuffle(coords)
    c = dev(coords)
    res = generate_kernel_map(c, c, (1, 1, 1), (3, 3, 3), kernel_dilation=dilation)
    assert np.array_equal(res.neighbor_table(len(coords)).cpu().numpy(),
                          km.kernel_map_found(coords, coords, (1, 1, 1), (3, 3, 3), dilation))
    i, o, f, _ = km.generate_kernel_map(coords, coords, (1, 1, 1), (3, 3, 3), dilation)
    assert_map_equal(res, i, o, f)
    coarse, _ = km.stride_coords(coords, (2, 2, 2))
    res2 = generate_kernel_map(c, dev(coarse), (2, 2, 2), (2, 2, 2), kernel_dilation=dilation)
    assert np.array_equal(res2.neighbor_table(len(coarse)).cpu().numpy(),
                          km.kernel_map_found(coords, coarse, (2, 2, 2), (2, 2, 2), dilation))
    check_device_status(DEV)


def test_expand_coords_matches_oracle_set():
    from warpconvnet_b200.geometry.coords.ops.expand import expand_coords
    scenes = [synthetic.room_scene(3000, 0.05, 700 + i, "sample") - 11 for i in range(2)]
    coords, offsets = synthetic.batch_scenes(scenes)
    for ks, dil in (((3, 3, 3), (1, 1, 1)), ((2, 2, 2), (1, 1, 1)), ((3, 1, 3), (2, 1, 1))):
        rows, offs = expand_coords(dev(coords.astype(np.int32)), ks, dil)
        want, want_off = km.expand_coords(coords, ks, dil)
        got = rows.cpu().numpy()
        assert np.array_equal(km.canonical_coords(got), want)
        assert np.array_equal(offs.numpy(), want_off)
        assert np.all(np.diff(got[:, 0]) >= 0)  # batch-sorted
    check_device_status(DEV)


# --------------------------------------------------------------------------- brick tables


def _sorted_voxels(coords, offsets):
    from warpconvnet_b200 import POINT_ORDERING, Voxels
    vox = Voxels(dev(coords[:, 1:]), torch.zeros(len(coords), 1, device=DEV), offsets=torch.from_numpy(np.asarray(offsets)))
    return vox.sort(POINT_ORDERING.MORTON_XYZ)


def test_brick_table_maps_match_oracle_on_every_level():
    """Morton-ordered rooms (negative coordinates, ragged batch): the 3x3x3 map, the 2x2x2 stride-2
    map and its transposed view come from the brick table on the finest level AND on its stride-2
    and stride-4 down-samplings (the sort's corner is a multiple of 16, so every level stays
    brick-ordered), bit-exact against the oracle."""
    from warpconvnet_b200.nn.functional.sparse_conv import strided_coordinates
    scenes = [synthetic.room_scene(n, 0.02, 510 + i, "raster_crop") - np.array([37, 5, 11], np.int32)
              for i, n in enumerate((30000, 700, 12000))]
    coords, offsets = synthetic.batch_scenes(scenes)
    level = _sorted_voxels(coords, offsets).batched_coordinates
    for depth in range(3):
        bt = level.bricks
        hdr = bt.header()
        c_dev = level.batch_indexed_coordinates.contiguous()
        c = c_dev.cpu().numpy()
        assert hdr["valid"] and 0 < hdr["num_bricks"] < len(c) and hdr["cap"] >= 4 * hdr["num_bricks"]
        res = generate_kernel_map(c_dev, c_dev, (1, 1, 1), (3, 3, 3), hashtable=level.hashmap, bricks=bt)
        assert np.array_equal(res.neighbor_table(len(c)).cpu().numpy(), km.kernel_map_found(c, c, (1, 1, 1), (3, 3, 3)))
        i, o, f, iden = km.generate_kernel_map(c, c, (1, 1, 1), (3, 3, 3))
        assert_map_equal(res, i, o, f)
        coarse = strided_coordinates(level, (2, 2, 2))
        cc_dev = coarse.batch_indexed_coordinates.contiguous()
        cc = cc_dev.cpu().numpy()
        assert np.array_equal(cc, km.stride_coords(c, (2, 2, 2))[0])
        down = generate_kernel_map(c_dev, cc_dev, (2, 2, 2), (2, 2, 2), hashtable=level.hashmap, bricks=bt)
        want = km.kernel_map_found(c, cc, (2, 2, 2), (2, 2, 2))
        assert np.array_equal(down.neighbor_table(len(cc)).cpu().numpy(), want)
        odd = generate_kernel_map(c_dev, cc_dev, (2, 2, 2), (3, 2, 4), hashtable=level.hashmap, bricks=bt)
        assert np.array_equal(odd.neighbor_table(len(cc)).cpu().numpy(), km.kernel_map_found(c, cc, (2, 2, 2), (3, 2, 4)))
        level = coarse
    check_device_status(DEV)


def test_brick_table_falls_back_when_rows_are_not_brick_ordered():
    """Generator (raster) order, rows with repeats, and a corner that does not match the sort:
    the build marks the table unusable and the same call answers from the voxel table."""
    from warpconvnet_b200.geometry.coords.search.brick_table import BrickTable
    xyz = synthetic.room_scene(20000, 0.02, 77, "raster_crop")
    coords = np.concatenate([np.zeros((len(xyz), 1), np.int32), xyz], 1)
    dup = np.concatenate([coords, coords[:300]], 0)
    srt = _sorted_voxels(coords, [0, len(coords)]).batched_coordinates
    shifted_origin = srt.morton_origin + torch.tensor([1, 0, 2], dtype=torch.int32, device=DEV)
    cases = [(coords, torch.from_numpy(coords[:, 1:].min(0).astype(np.int32)).to(DEV)),
             (dup, torch.from_numpy(dup[:, 1:].min(0).astype(np.int32)).to(DEV)),
             (srt.batch_indexed_coordinates.cpu().numpy(), shifted_origin)]
    for rows, origin in cases:
        c_dev = dev(rows)
        ht = TorchHashTable.from_keys(c_dev)
        bt = BrickTable(c_dev, origin, ht)
        assert not bt.header()["valid"]
        want = km.kernel_map_found(rows, rows, (1, 1, 1), (3, 3, 3))
        res = generate_kernel_map(c_dev, c_dev, (1, 1, 1), (3, 3, 3), hashtable=ht, bricks=bt)
        assert np.array_equal(res.neighbor_table(len(rows)).cpu().numpy(), want)
        # a stand-by voxel table (insert kernels that only work when the bricks are unusable) was filled
        lone = BrickTable(c_dev, origin)
        res = generate_kernel_map(c_dev, c_dev, (1, 1, 1), (3, 3, 3), hashtable=lone.hashtable, bricks=lone)
        assert np.array_equal(res.neighbor_table(len(rows)).cpu().numpy(), want)
    # a sorted set about its own corner is usable whatever the corner's parity
    own = srt.batch_indexed_coordinates.contiguous()
    assert BrickTable(own, srt.morton_origin, srt.hashmap).header()["valid"]
    check_device_status(DEV)


def test_standby_voxel_table_is_filled_when_something_probes_it():
    """With usable bricks the voxel table behind them is left unbuilt (its buffer is poisoned here to
    make that visible); a direct search, a dilated map and a custom-centred map fill it first."""
    from warpconvnet_b200.geometry.coords.search.brick_table import BrickTable
    xyz = synthetic.room_scene(15000, 0.02, 78, "raster_crop")
    coords = np.concatenate([np.zeros((len(xyz), 1), np.int32), xyz], 1)
    srt = _sorted_voxels(coords, [0, len(coords)]).batched_coordinates
    own = srt.batch_indexed_coordinates.contiguous()
    rows = own.cpu().numpy()
    for probe in ("map", "search", "dilated"):
        bt = BrickTable(own, srt.morton_origin)
        ht = bt.hashtable
        assert bt.header()["valid"] and ht._standby
        ht._table.fill_(0x5A)  # whatever the skipped kernels left behind must not matter
        if probe == "map":
            res = generate_kernel_map(own, own, (1, 1, 1), (3, 3, 3), hashtable=ht, bricks=bt)
            assert ht._standby  # still not needed
            got, want = res.neighbor_table(len(rows)).cpu().numpy(), km.kernel_map_found(rows, rows, (1, 1, 1), (3, 3, 3))
        elif probe == "search":
            got, want = ht.search(own).cpu().numpy(), np.arange(len(rows), dtype=np.int32)
        else:
            res = generate_kernel_map(own, own, (1, 1, 1), (3, 3, 3), kernel_dilation=(2, 2, 2), hashtable=ht, bricks=bt)
            got = res.neighbor_table(len(rows)).cpu().numpy()
            want = km.kernel_map_found(rows, rows, (1, 1, 1), (3, 3, 3), kernel_dilation=(2, 2, 2))
        assert np.array_equal(got, want), probe
        assert ht._standby == (probe == "map")
    # IntCoords hands out the pair: the table of sorted coordinates is the stand-by of their bricks
    assert srt.hashmap is srt.bricks.hashtable
    check_device_status(DEV)


def test_pyramid_in_one_sync_equals_chained_levels(monkeypatch):
    """The coordinate pyramid computed from the finest rows with one read-back (small batches) gives,
    level by level, the rows, order and batch offsets of chaining stride_coords, and both equal the
    oracle."""
    import warpconvnet_b200.nn.functional.sparse_conv as F
    scenes = [synthetic.room_scene(n, 0.02, 530 + i, "raster_crop") - np.array([3, 41, 7], np.int32)
              for i, n in enumerate((20000, 300, 9000))]
    coords, offsets = synthetic.batch_scenes(scenes)
    fast = _sorted_voxels(coords, offsets)
    levels_fast = F.prefetch_strided_coordinates(fast, [2, 2, 2, 2])
    monkeypatch.setattr(F, "PYRAMID_ONE_SYNC_MAX_ROWS", 0)
    slow = _sorted_voxels(coords, offsets)
    levels_slow = F.prefetch_strided_coordinates(slow, [2, 2, 2, 2])
    want = fast.batch_indexed_coordinates.cpu().numpy()
    for a, b in zip(levels_fast, levels_slow):
        want, want_off = km.stride_coords(want, (2, 2, 2))
        assert np.array_equal(a.batch_indexed_coordinates.cpu().numpy(), want)
        assert np.array_equal(b.batch_indexed_coordinates.cpu().numpy(), want)
        assert np.array_equal(a.offsets.numpy(), want_off) and np.array_equal(b.offsets.numpy(), want_off)
        assert torch.equal(a.morton_origin, b.morton_origin) and a.bricks.header()["valid"]
    check_device_status(DEV)
