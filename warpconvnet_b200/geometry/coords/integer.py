"""``IntCoords``: integer voxel coordinates of a batch with a tensor stride and a
lazily built hash table (warpconvnet/geometry/coords/integer.py:19-105)."""
from __future__ import annotations

from typing import List, Optional, Tuple, Union

import torch
from torch import Tensor

from ...utils.ntuple import ntuple
from ..base.batched import Coords, _as_cpu_offsets, list_to_cat_tensor
from .ops.batch_index import batch_indexed_coordinates
from .search.torch_hashmap import TorchHashTable


class IntCoords(Coords):
    def __init__(self, batched_tensor: Union[List[Tensor], Tensor], offsets=None,
                 voxel_size: Optional[float] = None, voxel_origin: Optional[Tensor] = None,
                 tensor_stride: Optional[Union[int, Tuple[int, ...]]] = None,
                 device: Optional[Union[str, torch.device]] = None):
        if isinstance(batched_tensor, (list, tuple)):
            assert offsets is None, "If batched_tensors is a list, offsets must be None."
            batched_tensor, offsets, _ = list_to_cat_tensor(batched_tensor)
        if offsets is None:
            offsets = [0, batched_tensor.shape[0]]
        if device is not None:
            batched_tensor = batched_tensor.to(device)
        self.offsets = _as_cpu_offsets(offsets)
        self.batched_tensor = batched_tensor
        self.voxel_size = voxel_size
        self.voxel_origin = voxel_origin
        self.tensor_stride = (ntuple(tensor_stride, ndim=batched_tensor.shape[1])
                              if tensor_stride is not None else None)
        # derived data (batch-indexed form, hash table), shared by reference between coordinate
        # objects that view the same rows (see share_derived)
        self._shared = {}
        self.check()

    def check(self):
        Coords.check(self)
        assert self.batched_tensor.dtype in (torch.int32, torch.int64), "Discrete coordinates must be integers"
        if self.tensor_stride is not None:
            assert isinstance(self.tensor_stride, (int, tuple))

    def to(self, device=None, dtype=None):
        if device is None:
            device = self.device
        return IntCoords(self.batched_tensor.to(device=device), self.offsets, self.voxel_size, self.voxel_origin,
                         self.tensor_stride)

    @property
    def _bcoords(self):
        return self._shared.get("bcoords")

    @_bcoords.setter
    def _bcoords(self, value):
        self._shared["bcoords"] = value

    def share_derived(self, other: "IntCoords") -> "IntCoords":
        """Use the same derived data as ``other``, which must hold the same rows."""
        self._shared = other._shared
        return self

    @property
    def batch_indexed_coordinates(self) -> Tensor:
        """[N, 4] (batch, x, y, z); built once per set of rows."""
        if self._shared.get("bcoords") is None:
            self._shared["bcoords"] = batch_indexed_coordinates(self.batched_tensor, self.offsets)
        return self._shared["bcoords"]

    @property
    def hashmap(self) -> TorchHashTable:
        """Hash table of the batch-indexed int32 coordinates; built once per set of rows."""
        if self._shared.get("hashmap") is None:
            if self._shared.get("morton_origin") is not None and self.batched_tensor.shape[1] == 3:
                self._shared["hashmap"] = self.bricks.hashtable  # a stand-by table, filled only if the bricks are unusable
            else:
                self._shared["hashmap"] = TorchHashTable.from_keys(self.batch_indexed_coordinates.to(torch.int32))
        return self._shared["hashmap"]

    @property
    def morton_origin(self) -> Optional[Tensor]:
        """int32 ``[3]`` device tensor: the corner from which the Morton codes these rows are sorted by
        were taken, or None when the rows are in no such order (as far as is known)."""
        return self._shared.get("morton_origin")

    @morton_origin.setter
    def morton_origin(self, value: Optional[Tensor]):
        self._shared["morton_origin"] = value

    @property
    def bricks(self):
        """Brick table of the batch-indexed coordinates (built once per set of rows), or None when
        the rows are not known to be Morton-ordered or are not 3-D."""
        if self._shared.get("morton_origin") is None or self.batched_tensor.shape[1] != 3:
            return None
        if self._shared.get("bricks") is None:
            from .search.brick_table import BrickTable
            self._shared["bricks"] = BrickTable(self.batch_indexed_coordinates.to(torch.int32),
                                                self._shared["morton_origin"], self._shared.get("hashmap"))
            self._shared["hashmap"] = self._shared["bricks"].hashtable
        return self._shared["bricks"]

    @property
    def stride(self):
        return self.tensor_stride

    def set_tensor_stride(self, tensor_stride: Union[int, Tuple[int, ...]]):
        self.tensor_stride = ntuple(tensor_stride, ndim=self.num_spatial_dims)

    def sort(self, ordering=None) -> "IntCoords":
        from .ops.serialization import POINT_ORDERING, encode
        ordering = ordering or POINT_ORDERING.MORTON_XYZ
        perm = encode(self.batched_tensor, batch_offsets=self.offsets, order=ordering, return_perm=True).perm
        return IntCoords(self.batched_tensor[perm], self.offsets, self.voxel_size, self.voxel_origin,
                         self.tensor_stride)

    def unique(self) -> "IntCoords":
        from .ops.stride import unique_strided_rows
        from .ops.batch_index import offsets_from_batch_index
        rows, _, _ = unique_strided_rows(self.batch_indexed_coordinates.to(torch.int32))
        return IntCoords(rows[:, 1:].to(self.batched_tensor.dtype), offsets_from_batch_index(rows[:, 0]),
                         self.voxel_size, self.voxel_origin, self.tensor_stride)
