"""``Voxels``: a batch of sparse voxel grids — integer coordinates, features,
per-batch offsets, tensor stride and the shared kernel-map cache
(warpconvnet/geometry/types/voxels.py:23-73, 255-303)."""
from __future__ import annotations

from typing import List, Optional, Tuple, Union

import torch
from torch import Tensor

from ..base.geometry import Geometry
from ..coords.integer import IntCoords
from ..coords.ops.batch_index import offsets_from_batch_index
from ..coords.ops.serialization import POINT_ORDERING, encode
from ..coords.ops.stride import unique_strided_rows
from ..coords.search.torch_hashmap import TorchHashTable
from ..features.cat import CatFeatures, to_batched_features


class Voxels(Geometry):
    def __init__(self, batched_coordinates: Union[List[Tensor], Tensor, IntCoords],
                 batched_features: Union[List[Tensor], Tensor, CatFeatures],
                 offsets: Optional[Tensor] = None, device: Optional[str] = None, **kwargs):
        tensor_stride = kwargs.pop("tensor_stride", None) or kwargs.pop("stride", None)
        if isinstance(batched_coordinates, list):
            assert isinstance(batched_features, list), "If coords is a list, features must be a list too."
            assert len(batched_coordinates) == len(batched_features)
            assert all(len(c) == len(f) for c, f in zip(batched_coordinates, batched_features))
            batched_coordinates = IntCoords(batched_coordinates, device=device, tensor_stride=tensor_stride)
        elif isinstance(batched_coordinates, Tensor):
            assert isinstance(batched_features, Tensor) and offsets is not None, \
                "If coordinate is a tensor, features must be a tensor and offsets must be provided."
            batched_coordinates = IntCoords(batched_coordinates, offsets=offsets, device=device,
                                            tensor_stride=tensor_stride)
        elif tensor_stride is not None:
            batched_coordinates.set_tensor_stride(tensor_stride)
        if isinstance(batched_features, list):
            batched_features = CatFeatures(batched_features, device=device)
        elif isinstance(batched_features, Tensor):
            batched_features = to_batched_features(batched_features, batched_coordinates.offsets, device=device)
        Geometry.__init__(self, batched_coordinates, batched_features, **kwargs)

    # -- coordinates
    @property
    def batch_indexed_coordinates(self) -> Tensor:
        return self.batched_coordinates.batch_indexed_coordinates

    @property
    def coordinate_hashmap(self) -> TorchHashTable:
        return self.batched_coordinates.hashmap

    @property
    def tensor_stride(self):
        return self.batched_coordinates.tensor_stride

    stride = tensor_stride

    def set_tensor_stride(self, tensor_stride: Union[int, Tuple[int, ...]]):
        self.batched_coordinates.set_tensor_stride(tensor_stride)

    @property
    def voxel_size(self):
        return self._extra_attributes.get("voxel_size", None)

    @property
    def ordering(self):
        return self._extra_attributes.get("ordering", None)

    # -- whole-tensor transforms
    def sort(self, ordering: POINT_ORDERING = POINT_ORDERING.MORTON_XYZ) -> "Voxels":
        """Rows of every batch item sorted by Morton code (voxels.py:255-267).

        For ``MORTON_XYZ`` on a CUDA device the codes are taken from the per-axis minimum rounded
        DOWN to a multiple of 16 (the reference subtracts the minimum itself,
        coords/ops/serialization.py:224-225; :func:`encode` and :func:`morton_code` still do).  Both are
        Morton orders of the same rows; with the rounded corner the 4x4x4 bricks of this
        coordinate set and of its stride-2, 4, 8 and 16 down-samplings are all aligned with the order,
        which is what lets the kernel maps of every level use a brick table."""
        if ordering == self.ordering:
            return self
        assert isinstance(ordering, POINT_ORDERING), f"Invalid ordering: {ordering}"
        origin = None
        coords = self.coordinate_tensor
        if ordering == POINT_ORDERING.MORTON_XYZ and coords.is_cuda and coords.shape[0] > 0 and coords.shape[1] == 3:
            lowest = coords.min(dim=0).values.to(torch.int32)
            origin = (torch.div(lowest, 16, rounding_mode="floor") * 16).contiguous()  # the corner the codes are taken from
        res = encode(coords, batch_offsets=self.offsets, order=ordering, return_perm=True, origin=origin)
        kwargs = self.extra_attributes
        kwargs["ordering"] = ordering
        kwargs["code"] = res.codes
        kwargs["perm"] = res.perm  # sorted = original[perm]
        kwargs.pop("_cache", None)  # cached maps index the old row order
        sorted_coords = IntCoords(coords[res.perm], self.offsets, tensor_stride=self.tensor_stride)
        if origin is not None:
            # rows sorted by the Morton code of (coords - origin): kernel maps may use a brick table
            sorted_coords.morton_origin = origin
        return self.__class__(batched_coordinates=sorted_coords,
                              batched_features=CatFeatures(self.feature_tensor[res.perm], self.offsets), **kwargs)

    def unique(self) -> "Voxels":
        """One voxel per distinct coordinate, keeping its first occurrence (voxels.py:269-276)."""
        rows, uidx, _ = unique_strided_rows(self.batch_indexed_coordinates.to(torch.int32))
        offsets = offsets_from_batch_index(rows[:, 0])
        kwargs = self.extra_attributes
        kwargs.pop("_cache", None)
        coords = IntCoords(self.coordinate_tensor[uidx.long()], offsets, tensor_stride=self.tensor_stride)
        feats = CatFeatures(self.feature_tensor[uidx.long()], offsets)
        return self.__class__(coords, feats, **kwargs)
