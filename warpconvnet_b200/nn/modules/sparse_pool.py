"""Pooling modules for ``Voxels`` (warpconvnet/nn/modules/sparse_pool.py:20-140)."""
from __future__ import annotations

from ...geometry.types.voxels import Voxels
from ..functional.sparse_pool import sparse_reduce, sparse_unpool
from .base_module import BaseSpatialModule


class SparsePool(BaseSpatialModule):
    """Reduce the features of every ``kernel_size`` window placed at multiples of ``stride``."""

    def __init__(self, kernel_size: int, stride: int, reduce: str = "max"):
        super().__init__()
        self.kernel_size = kernel_size
        self.stride = stride
        self.reduce = reduce

    def __repr__(self):
        return f"{self.__class__.__name__}(kernel_size={self.kernel_size}, stride={self.stride}, reduce={self.reduce})"

    def forward(self, st: Voxels):
        return sparse_reduce(st, self.kernel_size, self.stride, self.reduce)


class SparseMaxPool(SparsePool):
    def __init__(self, kernel_size: int, stride: int):
        super().__init__(kernel_size, stride, "max")


class SparseMinPool(SparsePool):
    def __init__(self, kernel_size: int, stride: int):
        super().__init__(kernel_size, stride, "min")


class SparseUnpool(BaseSpatialModule):
    """Copy pooled features back to the resolution they were pooled from."""

    def __init__(self, kernel_size: int, stride: int, concat_unpooled_st: bool = True):
        super().__init__()
        self.kernel_size = kernel_size
        self.stride = stride
        self.concat_unpooled_st = concat_unpooled_st

    def forward(self, st: Voxels, unpooled_st: Voxels):
        return sparse_unpool(st, unpooled_st, self.kernel_size, self.stride, self.concat_unpooled_st)
