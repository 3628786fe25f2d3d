"""Morton ordering of voxel coordinates (warpconvnet/geometry/coords/ops/serialization.py:60-254).

``morton_code`` subtracts the per-axis minimum, permutes the axes for the
non-XYZ orders and interleaves 3 x <=21-bit integers (x in bit 0).  ``encode``
returns the codes and, on request, the permutation that sorts each batch
segment by code.
"""
from __future__ import annotations

import ctypes
import enum
from typing import NamedTuple, Optional, Union

import torch
from torch import Tensor

from ...._native import check, lib, ptr, stream_ptr


class POINT_ORDERING(enum.Enum):
    RANDOM = "random"
    MORTON_XYZ = "morton_xyz"
    MORTON_XZY = "morton_xzy"
    MORTON_YXZ = "morton_yxz"
    MORTON_YZX = "morton_yzx"
    MORTON_ZXY = "morton_zxy"
    MORTON_ZYX = "morton_zyx"


STR2POINT_ORDERING = {m.value: m for m in POINT_ORDERING}

POINT_ORDERING_TO_MORTON_PERMUTATIONS = {
    POINT_ORDERING.MORTON_XYZ: [0, 1, 2],
    POINT_ORDERING.MORTON_XZY: [0, 2, 1],
    POINT_ORDERING.MORTON_YXZ: [1, 0, 2],
    POINT_ORDERING.MORTON_YZX: [1, 2, 0],
    POINT_ORDERING.MORTON_ZXY: [2, 0, 1],
    POINT_ORDERING.MORTON_ZYX: [2, 1, 0],
}


class SerializationResult(NamedTuple):
    codes: Tensor
    perm: Optional[Tensor] = None
    inverse_perm: Optional[Tensor] = None
    counts: Optional[Tensor] = None


@torch.no_grad()
def morton_code(coords: Tensor, threads_per_block: int = 256,
                order: Union[POINT_ORDERING, str] = POINT_ORDERING.MORTON_XYZ,
                origin: Optional[Tensor] = None) -> Tensor:
    """int64 Morton codes of ``coords [N,3]`` (integer voxel coordinates).  ``origin`` (an addition
    to the reference signature): the per-axis minimum of ``coords`` as an int32 ``[3]`` device
    tensor, when the caller already has it."""
    if isinstance(order, str):
        order = POINT_ORDERING(order)
    assert order in POINT_ORDERING_TO_MORTON_PERMUTATIONS, f"Order '{order}' not supported for morton code"
    if coords.shape[0] == 0:
        return torch.empty(0, dtype=torch.int64)
    assert coords.shape[1] == 3, "coords must be [N, 3]"
    assert coords.is_cuda, "coords must be on a CUDA device"
    perm = POINT_ORDERING_TO_MORTON_PERMUTATIONS[order]
    c = coords.to(torch.int32)
    if perm != [0, 1, 2]:
        c = c[:, perm]
    c = c.contiguous()
    if origin is not None and perm == [0, 1, 2]:
        mins = origin.to(torch.int32).contiguous()
    else:
        mins = c.min(dim=0).values.contiguous()  # stays on the device: no host synchronisation
    codes = torch.empty(c.shape[0], dtype=torch.int64, device=c.device)
    check(lib().wcn_morton20(ptr(c), c.shape[0], 3, 0, ptr(mins), ptr(codes), stream_ptr(c.device)),
          "wcn_morton20")
    return codes


@torch.no_grad()
def encode(grid_coord: Tensor, batch_offsets: Optional[Tensor] = None,
           order: Union[POINT_ORDERING, str] = POINT_ORDERING.MORTON_XYZ, return_perm: bool = False,
           return_inverse: bool = False, size=None, num_buckets=None, origin: Optional[Tensor] = None):
    if isinstance(order, str):
        order = STR2POINT_ORDERING[order.lower()]
    if grid_coord.shape[0] == 0:
        codes = torch.empty(0, dtype=torch.int64)
    elif order in POINT_ORDERING_TO_MORTON_PERMUTATIONS:
        codes = morton_code(grid_coord[:, -3:], order=order, origin=origin)
    elif order == POINT_ORDERING.RANDOM:
        codes = torch.randperm(grid_coord.shape[0], device=grid_coord.device)
    else:
        raise NotImplementedError(f"Order '{order}' not supported at the moment")
    if not return_perm and not return_inverse:
        return codes
    if codes.shape[0] == 0:
        e = torch.empty(0, dtype=torch.int64)
        return SerializationResult(codes, e if return_perm else None, e if return_inverse else None)
    if batch_offsets is not None and len(batch_offsets) > 2:
        # sort by code inside each batch segment: stable sort by code, then stable sort by batch
        from .batch_index import batch_index_on
        # (the narrowest batch key: the radix sort behind argsort runs one pass per key byte)
        nb = len(batch_offsets) - 1
        seg_dtype = torch.uint8 if nb <= 256 else torch.int16 if nb < 2 ** 15 else torch.int64
        seg = batch_index_on(batch_offsets, codes.shape[0], codes.device, seg_dtype)
        by_code = torch.argsort(codes, stable=True)
        perm = by_code[torch.argsort(seg[by_code], stable=True)]
    else:
        perm = torch.argsort(codes, stable=True)
    inverse = None
    if return_inverse:
        inverse = torch.empty_like(perm)
        inverse[perm] = torch.arange(len(perm), device=perm.device)
    return SerializationResult(codes=codes, perm=perm, inverse_perm=inverse)
