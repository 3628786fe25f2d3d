"""The oracle against the reference: golden vectors generated from the reference
itself, and (when oracle/_ref is built) the reference's kernels compiled for the host."""
import numpy as np
import pytest
import torch

from oracle import kernel_map as km
from oracle import ref_loader
from oracle import sparse_conv as osc
from warpconvnet_b200.datasets import synthetic

from conftest import rel_l2


def test_kernel_offsets_match_reference(golden):
    g = golden("kernel_offsets.npz")
    assert np.array_equal(km.kernel_offsets_from_size((3, 3, 3)), g["k333"])
    assert np.array_equal(km.kernel_offsets_from_size((2, 2, 2)), g["k222"])
    assert np.array_equal(km.kernel_offsets_from_size((3, 1, 2)), g["k312"])
    assert np.array_equal(km.kernel_offsets_from_size((3, 3, 3), (2, 2, 2)), g["k333_d2"])
    # first / last rows of the 3x3x3 window: last axis fastest, centred
    assert g["k333"][0].tolist() == [0, -1, -1, -1] and g["k333"][26].tolist() == [0, 1, 1, 1]
    assert g["k333"][1].tolist() == [0, -1, -1, 0]
    assert g["k222"][0].tolist() == [0, 0, 0, 0] and g["k222"][7].tolist() == [0, 1, 1, 1]


def test_hash_search_matches_reference(golden):
    g = golden("kmap_small.npz")
    assert np.array_equal(km.hash_search(g["coords"], g["queries"]), g["search"])
    assert (g["search"][:400] >= 0).all() and (g["search"][400:] == -1).all()


@pytest.mark.parametrize("tag,stride,ks", [("333", (1, 1, 1), (3, 3, 3)), ("222", (2, 2, 2), (2, 2, 2)),
                                            ("312", (1, 1, 1), (3, 1, 2))])
def test_kernel_map_matches_reference(golden, tag, stride, ks):
    g = golden("kmap_small.npz")
    out_coords = g["out_coords"] if tag == "222" else g["coords"]
    i, o, f, iden = km.generate_kernel_map(g["coords"], out_coords, stride, ks)
    assert np.array_equal(i, g["in" + tag]) and np.array_equal(o, g["out" + tag]) and np.array_equal(f, g["off" + tag])
    assert iden == (13 if tag == "333" else None)


def test_transposed_map_matches_reference(golden):
    g = golden("kmap_small.npz")
    i, o, f, iden = km.transposed_kernel_map(g["out_coords"], g["coords"], (2, 2, 2), (2, 2, 2))
    assert np.array_equal(i, g["tr_in"]) and np.array_equal(o, g["tr_out"]) and np.array_equal(f, g["tr_off"])
    assert iden is None
    # every fine voxel has exactly one coarse parent
    assert len(o) == len(g["coords"]) and len(np.unique(o)) == len(o)


def test_stride_coords_set_and_offsets(golden):
    g = golden("kmap_small.npz")
    out, offsets = km.stride_coords(g["coords"], (2, 2, 2))
    assert np.array_equal(out, g["out_coords"])
    ref_set = np.unique(np.floor_divide(g["coords"], np.array([1, 2, 2, 2])), axis=0)
    assert np.array_equal(km.canonical_coords(out), ref_set)
    assert len(offsets) == 4 and offsets[-1] == len(out) and len(out) < len(g["coords"])
    assert (np.diff(out[:, 0]) >= 0).all()


def test_morton_matches_reference(golden):
    g = golden("kmap_small.npz")
    assert np.array_equal(km.morton_code(g["morton_xyz"], subtract_min=False), g["morton"])
    order = np.argsort(g["morton"], kind="stable")
    assert (np.diff(g["morton"][order]) >= 0).all()


def test_explicit_gemm_matches_reference_small(golden):
    g, c = golden("kmap_small.npz"), golden("conv_small.npz")
    x = torch.from_numpy(c["x"])
    n = len(g["coords"])
    y = osc.explicit_gemm_forward(x, torch.from_numpy(c["w333"]), g["in333"], g["out333"], g["off333"], 13, n)
    assert np.array_equal(y.numpy(), c["y333"])
    y2 = osc.explicit_gemm_forward(x, torch.from_numpy(c["w222"]), g["in222"], g["out222"], g["off222"], None,
                                   len(g["out_coords"]))
    assert np.array_equal(y2.numpy(), c["y222"])
    y3 = osc.explicit_gemm_forward(y2, torch.from_numpy(c["wtr"]), g["tr_in"], g["tr_out"], g["tr_off"], None, n)
    assert np.array_equal(y3.numpy(), c["ytr"])


def test_config1_matches_reference(golden):
    """Single SparseConv3d layer, 20 000 voxels of [0,64)^3, C=32, fp32."""
    g = golden("conv_config1.npz")
    xyz = synthetic.random_cells(20000, 64, seed=0)
    coords = np.concatenate([np.zeros((len(xyz), 1), np.int32), xyz], 1)
    i, o, f, iden = km.generate_kernel_map(coords, coords, (1, 1, 1), (3, 3, 3))
    assert np.array_equal(f, g["offsets"]) and int(f[-1]) == 58192
    assert int(i.astype(np.int64).sum()) == int(g["in_maps_sum"]) and int(o.astype(np.int64).sum()) == int(g["out_maps_sum"])
    x = np.random.default_rng(0).standard_normal((20000, 32)).astype(np.float32)
    y = osc.explicit_gemm_forward(torch.from_numpy(x), torch.from_numpy(g["weight"]), i, o, f, iden, 20000).numpy()
    assert rel_l2(y[g["rows"]], g["y_rows"]) < 1e-6
    assert np.allclose(y.astype(np.float64).sum(0), g["y_colsum"], rtol=1e-6, atol=1e-6)
    assert abs((y.astype(np.float64) ** 2).sum() - float(g["y_sqnorm"])) / float(g["y_sqnorm"]) < 1e-9


def test_probe_sequence_restatement_tiny():
    rng = np.random.default_rng(3)
    keys = rng.integers(-5, 5, size=(40, 4)).astype(np.int32)
    keys = np.unique(keys, axis=0)
    q = np.concatenate([keys[:10], keys[:10] + np.array([0, 50, 0, 0], np.int32)])
    for method in ("city", "fnv1a", "murmur"):
        t = km.ProbeTable(keys, method)
        assert np.array_equal(t.search(q), km.hash_search(keys, q))


def test_dilated_and_recentred_maps_match_reference(golden):
    """Dilated windows and a custom window centre: the oracle's found[K, M] against the reference's
    offset-list kernel (discrete_kernels.cu:129-180) run on its own offset lists."""
    g = golden("kmap_extra.npz")
    dil, ctr = tuple(g["dilation"]), tuple(g["center"])
    assert np.array_equal(km.kernel_offsets_from_size((3, 3, 3), dil), g["offs_d"])
    assert np.array_equal(km.kernel_offsets_from_size((3, 2, 3), None, ctr), g["offs_c"])
    assert np.array_equal(km.kernel_map_found(g["coords"], g["coords"], (1, 1, 1), (3, 3, 3), dil), g["found_d"])
    assert np.array_equal(km.kernel_map_found(g["coords"], g["coords"], (1, 1, 1), (3, 2, 3), None, ctr), g["found_c"])
    assert np.array_equal(km.kernel_map_found(g["coords"], g["coarse"], (2, 2, 2), (3, 3, 3), dil), g["found_ds"])
    assert (g["found_d"] >= 0).sum() > len(g["coords"])  # the fixture is not trivially empty


def test_expand_coords_matches_reference(golden):
    """Output support of a generative convolution: the oracle's set against the reference's
    expand_coords loop run with its own hash-search kernel."""
    g = golden("kmap_extra.npz")
    out, offsets = km.expand_coords(g["coords"], (3, 3, 3), (1, 2, 1))
    assert np.array_equal(out, g["grown"])
    assert offsets[-1] == len(out) and len(out) > len(g["coords"])


@pytest.mark.parametrize("red", ["max", "min", "mean", "sum", "mul", "var", "std"])
def test_window_reduce_matches_reference(golden, red):
    """Pooling: the oracle's window_reduce against the reference's to_csr + row_reduction
    (ops/reductions.py:36-70) with torch.segment_reduce standing in for torch_scatter.segment_csr."""
    g = golden("kmap_extra.npz")
    got = osc.window_reduce(g["feats"], g["in222"], g["out222"], len(g["coarse"]), red)
    # the reference evaluates mean(x^2) - mean(x)^2 in fp32 (cancellation); the root magnifies that
    assert np.allclose(got, g["pool_" + red], rtol=1e-5, atol=2e-4 if red == "std" else 1e-5)


# -- against the reference's kernels compiled for the host (built where the reference tree is present)

needs_ref = pytest.mark.skipif(not ref_loader.have_compiled_reference(), reason="oracle/_ref not built")


@needs_ref
@pytest.mark.parametrize("method", ["city", "fnv1a", "murmur"])
def test_oracle_vs_compiled_reference(method):
    rng = np.random.default_rng(11)
    scenes = [synthetic.room_scene(4000, 0.05, 300 + s, "sample") - np.array([50, 50, 0], np.int32) for s in range(3)]
    coords, _ = synthetic.batch_scenes(scenes)
    a = km.generate_kernel_map(coords, coords, (1, 1, 1), (3, 3, 3))
    b = ref_loader.ref_generate_kernel_map(coords, coords, (1, 1, 1), (3, 3, 3), method)
    for x, y in zip(a[:3], b):
        assert np.array_equal(x, y)
    out, _ = km.stride_coords(coords, (2, 2, 2))
    a = km.generate_kernel_map(coords, out, (2, 2, 2), (2, 2, 2))
    b = ref_loader.ref_generate_kernel_map(coords, out, (2, 2, 2), (2, 2, 2), method)
    for x, y in zip(a[:3], b):
        assert np.array_equal(x, y)
    t = ref_loader.RefHashTable(coords[:300], method)
    p = km.ProbeTable(coords[:300], method)
    assert p.marker == t.table[:, 0].tolist() and p.value == t.table[:, 1].tolist()
    assert np.array_equal(km.morton_code(coords[:, 1:] - coords[:, 1:].min(0), False),
                          ref_loader.ref_morton20(coords[:, 1:] - coords[:, 1:].min(0)))


@needs_ref
def test_reference_with_duplicates_returns_a_duplicate():
    """With repeated keys the reference returns SOME row holding the key; the oracle the first."""
    rng = np.random.default_rng(5)
    base = rng.integers(0, 6, size=(200, 4)).astype(np.int32)
    t = ref_loader.RefHashTable(base, "city")
    r = t.search(base)
    assert (r >= 0).all() and np.array_equal(base[r], base)
    assert np.array_equal(base[km.hash_search(base, base)], base)
