"""Pooling and un-pooling of ``Voxels`` (warpconvnet/nn/functional/sparse_pool.py:25-179).

``sparse_reduce`` reduces every ``kernel_size`` window placed at multiples of ``stride`` onto the
strided coordinate set; the kernel map is the one a strided convolution of the same geometry
uses and is shared with it through the map cache.  ``sparse_unpool`` copies each pooled row
back to the rows it was pooled from.
"""
from __future__ import annotations

from typing import Optional, Tuple, Union

import torch

from ...geometry.coords.ops.serialization import POINT_ORDERING
from ...geometry.coords.search.cache import IntSearchCacheKey
from ...geometry.types.voxels import Voxels
from ...ops.reductions import REDUCTIONS, neighbor_reduction
from ...utils.ntuple import ntuple
from .sparse_conv import STRIDED_CONV_MODE, generate_output_coords_and_kernel_map, strided_coordinates


def sparse_reduce(voxels: Voxels, kernel_size: Union[int, Tuple[int, ...]],
                  stride: Optional[Union[int, Tuple[int, ...]]] = None,
                  reduction: Union[REDUCTIONS, str] = REDUCTIONS.MAX,
                  order: POINT_ORDERING = POINT_ORDERING.RANDOM) -> Voxels:
    """Window reduction (max / min / mean / sum / mul / var / std / random) onto the strided coordinates."""
    if isinstance(reduction, str):
        reduction = REDUCTIONS(reduction)
    if stride is None:
        stride = kernel_size
    nd = voxels.num_spatial_dims
    stride, kernel_size = ntuple(stride, ndim=nd), ntuple(kernel_size, ndim=nd)
    in_tensor_stride = voxels.tensor_stride or ntuple(1, ndim=nd)
    out_tensor_stride = tuple(o * s for o, s in zip(stride, in_tensor_stride))
    if order != POINT_ORDERING.RANDOM:
        raise NotImplementedError("sparse_reduce keeps the first-occurrence order of the strided coordinates")
    # same key, same map as a strided convolution of this geometry (sparse_pool.py:52-80)
    _, _, kernel_map = generate_output_coords_and_kernel_map(
        voxels, kernel_size, ntuple(1, ndim=nd), stride, False, False, None, STRIDED_CONV_MODE.STRIDE_ONLY, order)
    out_ic = (strided_coordinates(voxels.batched_coordinates, stride) if any(s != 1 for s in stride)
              else voxels.batched_coordinates)
    num_out = out_ic.batched_tensor.shape[0]
    out = neighbor_reduction(voxels.feature_tensor, kernel_map, num_out, reduction)
    if out_ic.tensor_stride is None:
        out_ic.tensor_stride = out_tensor_stride
    return voxels.replace(batched_coordinates=out_ic, batched_features=out, tensor_stride=out_tensor_stride)


def sparse_max_pool(voxels: Voxels, kernel_size, stride=None) -> Voxels:
    return sparse_reduce(voxels, kernel_size, stride, reduction=REDUCTIONS.MAX)


def sparse_avg_pool(voxels: Voxels, kernel_size, stride=None) -> Voxels:
    return sparse_reduce(voxels, kernel_size, stride, reduction=REDUCTIONS.MEAN)


def sparse_unpool(pooled_voxels: Voxels, unpooled_voxels: Voxels, kernel_size, stride,
                  concat_unpooled_voxels: bool = False) -> Voxels:
    """Every row of ``unpooled_voxels`` receives the features of the pooled row it went into; the map
    is the one ``sparse_reduce`` left in the shared cache (windows must not overlap)."""
    nd = pooled_voxels.num_spatial_dims
    stride, kernel_size = ntuple(stride, ndim=nd), ntuple(kernel_size, ndim=nd)
    key = IntSearchCacheKey(kernel_size=kernel_size, kernel_dilation=ntuple(1, ndim=nd), transposed=False,
                            generative=False, stride_mode=str(STRIDED_CONV_MODE.STRIDE_ONLY),
                            skip_symmetric_kernel_map=False, in_offsets=unpooled_voxels.offsets,
                            out_offsets=pooled_voxels.offsets)
    assert pooled_voxels.cache is not None
    kernel_map = pooled_voxels.cache.get(key)
    assert kernel_map is not None
    assert all(k <= s for k, s in zip(kernel_size, stride)), "un-pooling needs non-overlapping windows"
    n = unpooled_voxels.coordinate_tensor.shape[0]
    up = kernel_map.swapped(num_in=n)
    # one neighbour per row: the sum is a copy, and its backward is the native sum over the pooling map
    rep = neighbor_reduction(pooled_voxels.feature_tensor, up, n, REDUCTIONS.SUM)
    if concat_unpooled_voxels:
        rep = torch.cat([unpooled_voxels.feature_tensor, rep], dim=-1)
    return unpooled_voxels.replace(batched_features=rep)
