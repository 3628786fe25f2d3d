"""Kernel-map cache shared by every tensor derived from one input
(warpconvnet/geometry/coords/search/cache.py:84-153).  The key holds the kernel
geometry and the per-batch voxel counts of both sides, never coordinates."""
from __future__ import annotations

from typing import Optional, Tuple

from torch import Tensor

from .search_results import IntSearchResult


def _offsets_tuple(offsets: Tensor) -> Tuple[int, ...]:
    """Batch offsets as a tuple of ints; remembered on the (CPU, never mutated) tensor object
    because the same offsets tensor is keyed once per layer of a network."""
    memo = offsets.__dict__.get("_wcn_tuple") if hasattr(offsets, "__dict__") else None
    if memo is None:
        memo = tuple(int(v) for v in offsets.detach().cpu().tolist())
        try:
            offsets.__dict__["_wcn_tuple"] = memo
        except Exception:  # pragma: no cover - tensors without a dict
            pass
    return memo


class IntSearchCacheKey:
    def __init__(self, kernel_size, kernel_dilation, transposed, generative, stride_mode,
                 skip_symmetric_kernel_map, in_offsets: Tensor, out_offsets: Tensor):
        self.kernel_size: Tuple[int, ...] = tuple(kernel_size)
        self.kernel_dilation: Tuple[int, ...] = tuple(kernel_dilation)
        self.transposed = bool(transposed)
        self.generative = bool(generative)
        self.stride_mode = str(stride_mode)
        self.skip_symmetric_kernel_map = bool(skip_symmetric_kernel_map)
        self.in_offsets = in_offsets
        self.out_offsets = out_offsets
        self._key = (self.kernel_size, self.kernel_dilation, self.transposed, self.generative, self.stride_mode,
                     self.skip_symmetric_kernel_map, _offsets_tuple(in_offsets), _offsets_tuple(out_offsets))

    def __hash__(self):
        return hash(self._key)

    def __eq__(self, other):
        return isinstance(other, IntSearchCacheKey) and self._key == other._key

    def __repr__(self):
        return (f"IntSearchCacheKey(kernel_size={self.kernel_size}, kernel_dilation={self.kernel_dilation}, "
                f"transposed={self.transposed}, generative={self.generative}, stride_mode={self.stride_mode}, "
                f"skip_symmetric_kernel_map={self.skip_symmetric_kernel_map}, num_in={self._key[-2][-1]}, "
                f"num_out={self._key[-1][-1]})")


class IntSearchCache(dict):
    def get(self, key: IntSearchCacheKey) -> Optional[IntSearchResult]:
        return super().get(key, None)

    def put(self, key: IntSearchCacheKey, value: IntSearchResult):
        super().__setitem__(key, value)

    def __repr__(self):
        return f"{self.__class__.__name__}({len(self)} keys)"
