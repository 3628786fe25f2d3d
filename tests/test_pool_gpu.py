"""GPU parity of pooling over kernel maps: ``sparse_reduce`` / ``sparse_unpool`` and the
``reduce_and_stride`` mode of the convolution against the oracle's restatement of the reference."""
import numpy as np
import pytest
import torch

from oracle import kernel_map as km
from oracle import sparse_conv as osc
from warpconvnet_b200 import (SPARSE_CONV_FWD_ALGO_MODE as ALGO, STRIDED_CONV_MODE, SparseMaxPool, SparseUnpool, Voxels,
                              sparse_reduce, sparse_unpool, spatially_sparse_conv)
from warpconvnet_b200._native import check_device_status
from warpconvnet_b200.datasets import synthetic

from conftest import rel_l2

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _scene(n, c, seed, dtype=torch.float32):
    scenes = [synthetic.room_scene(n, 0.04, seed + i, "sample") - 17 for i in range(2)]
    coords, offsets = synthetic.batch_scenes(scenes)
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(len(coords), c, generator=g).to(dtype)
    vox = Voxels(torch.from_numpy(coords[:, 1:].copy()).to(DEV), x.to(DEV), offsets=torch.from_numpy(offsets))
    return coords.astype(np.int32), x, vox


@pytest.mark.parametrize("reduction", ["max", "min", "mean", "sum", "mul", "var", "std"])
@pytest.mark.parametrize("c", [7, 32])
def test_sparse_reduce_matches_oracle(reduction, c):
    coords, x, vox = _scene(6000, c, 61)
    if reduction == "mul":
        x = x * 0.5 + 1.0
        vox = vox.replace(batched_features=x.to(DEV))
    out = sparse_reduce(vox, kernel_size=2, stride=2, reduction=reduction)
    check_device_status(DEV)
    ref_c, ref_off = km.stride_coords(coords, (2, 2, 2))
    i, o, f, _ = km.generate_kernel_map(coords, ref_c, (2, 2, 2), (2, 2, 2))
    want = osc.window_reduce(x.numpy(), i, o, len(ref_c), reduction)
    assert np.array_equal(out.batch_indexed_coordinates.cpu().numpy(), ref_c)
    assert np.array_equal(out.offsets.numpy(), ref_off)
    assert out.tensor_stride == (2, 2, 2)
    tol = 1e-4 if reduction in ("var", "std") else 1e-6
    assert rel_l2(out.feature_tensor.cpu().numpy(), want) < tol
    if reduction in ("max", "min"):
        assert np.array_equal(out.feature_tensor.cpu().numpy(), want.astype(np.float32))


def test_overlapping_windows_fp16_and_random():
    coords, x, vox = _scene(5000, 16, 62, torch.float16)
    out = sparse_reduce(vox, kernel_size=3, stride=2, reduction="max")
    ref_c, _ = km.stride_coords(coords, (2, 2, 2))
    i, o, f, _ = km.generate_kernel_map(coords, ref_c, (2, 2, 2), (3, 3, 3))
    want = osc.window_reduce(x.float().numpy(), i, o, len(ref_c), "max")
    assert np.array_equal(out.feature_tensor.float().cpu().numpy(), want.astype(np.float32))
    # random: every output row is one of the rows of its window
    rnd = sparse_reduce(vox, kernel_size=2, stride=2, reduction="random").feature_tensor.float().cpu().numpy()
    i2, o2, _, _ = km.generate_kernel_map(coords, ref_c, (2, 2, 2), (2, 2, 2))
    lo = osc.window_reduce(x.float().numpy(), i2, o2, len(ref_c), "min")
    hi = osc.window_reduce(x.float().numpy(), i2, o2, len(ref_c), "max")
    assert np.all(rnd >= lo - 1e-6) and np.all(rnd <= hi + 1e-6)
    check_device_status(DEV)


@pytest.mark.parametrize("concat", [True, False])
def test_unpool_copies_parents_back(concat):
    coords, x, vox = _scene(4000, 5, 63)
    pooled = SparseMaxPool(2, 2)(vox)
    up = SparseUnpool(2, 2, concat_unpooled_st=concat)(pooled, vox)
    ref_c, _ = km.stride_coords(coords, (2, 2, 2))
    i, o, f, _ = km.generate_kernel_map(coords, ref_c, (2, 2, 2), (2, 2, 2))
    parent = np.empty(len(coords), dtype=np.int64)
    parent[i] = o
    want = pooled.feature_tensor.cpu().numpy()[parent]
    got = up.feature_tensor.cpu().numpy()
    if concat:
        assert got.shape[1] == 10 and np.array_equal(got[:, :5], x.numpy()) and np.array_equal(got[:, 5:], want)
    else:
        assert np.array_equal(got, want)
    assert up.coordinate_tensor.shape[0] == len(coords)


def test_reduce_and_stride_convolution():
    """stride_mode=reduce_and_stride: pool the stride window (max), then a stride-1 convolution on the
    pooled tensor (warpconvnet/nn/functional/sparse_conv.py:1753-1767)."""
    coords, x, vox = _scene(5000, 8, 64)
    g = torch.Generator().manual_seed(3)
    w = torch.randn(27, 8, 12, generator=g) * 0.2
    with torch.no_grad():
        y = spatially_sparse_conv(vox, w.to(DEV), 3, stride=2, stride_mode=STRIDED_CONV_MODE.REDUCE_AND_STRIDE,
                                  stride_reduce="max", fwd_algo=ALGO.IMPLICIT_GEMM)
    ref_c, _ = km.stride_coords(coords, (2, 2, 2))
    i, o, f, _ = km.generate_kernel_map(coords, ref_c, (2, 2, 2), (2, 2, 2))
    pooled = osc.window_reduce(x.numpy(), i, o, len(ref_c), "max").astype(np.float32)
    i3, o3, f3, iden = km.generate_kernel_map(ref_c, ref_c, (1, 1, 1), (3, 3, 3))
    want = osc.explicit_gemm_forward(torch.from_numpy(pooled), w, i3, o3, f3, iden, len(ref_c)).numpy()
    assert np.array_equal(y.batch_indexed_coordinates.cpu().numpy(), ref_c)
    assert y.tensor_stride == (2, 2, 2)
    assert rel_l2(y.feature_tensor.cpu().numpy(), want) < 1e-4
    check_device_status(DEV)
