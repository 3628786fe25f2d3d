"""``BrickTable``: occupancy of 4x4x4 bricks of a Morton-ordered coordinate set.

An addition to the reference's search structures (it has none for ordered inputs): when the rows of
a coordinate set are sorted by Morton code — ``Voxels.sort`` — the rows of every 4x4x4 brick are
consecutive and ordered inside the brick, so one entry per brick (key, 64-bit occupancy mask, first
row) locates every voxel of it.  ``generate_kernel_map`` then answers a whole 3x3x3 or 2x2x2
window from at most eight entries instead of one hash probe per offset.  Whether the rows really
are brick-ordered is checked on the device while the table is built; if not, the search falls back
to the voxel hash table inside the same kernel, so callers never have to ask and results are
identical either way.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from ...._native import check, lib, ptr, query_bytes, stream_ptr
from .torch_hashmap import HashMethod, TorchHashTable


class BrickTable:
    def __init__(self, keys: Tensor, origin: Optional[Tensor], hashtable: Optional[TorchHashTable] = None,
                 hash_method: HashMethod = HashMethod.CITY):
        """``keys``: int32 ``[N, 4]`` rows (batch, x, y, z) on a CUDA device; ``origin``: int32 ``[3]`` on
        the same device, the corner the Morton codes were taken from (bricks are aligned to it), or
        None for the coordinate origin.  ``hashtable``: a voxel table already built over ``keys``; without
        one, a stand-by table is made whose insert kernels only do work when this brick table turns
        out unusable (``TorchHashTable.insert(standby_for=...)``)."""
        assert keys.is_cuda and keys.dtype == torch.int32 and keys.ndim == 2 and keys.shape[1] == 4
        assert hashtable is None or len(hashtable.vector_keys) == keys.shape[0], "hashtable was built over other keys"
        keys = keys.contiguous()
        dev = keys.device
        if origin is not None:
            origin = origin.to(device=dev, dtype=torch.int32).contiguous()
            assert origin.shape == (3,)
        self.keys, self.origin, self.hashtable = keys, origin, hashtable
        self._table = torch.empty(query_bytes("wcn_brick_table_bytes", keys.shape[0]), dtype=torch.uint8, device=dev)
        check(lib().wcn_brick_build(ptr(keys), keys.shape[0], ptr(origin), ptr(self._table), stream_ptr(dev)),
              "wcn_brick_build")
        if hashtable is None:
            self.hashtable = TorchHashTable.from_keys(keys, hash_method=hash_method, standby_for=self)

    @property
    def device(self) -> torch.device:
        return self._table.device

    def header(self) -> dict:
        """(synchronises) what the build found: slots in use, whether the rows were brick-ordered,
        number of bricks."""
        h = self._table[:32].view(torch.int32).cpu().tolist()
        return {"cap": h[0], "valid": bool(h[1]), "num_bricks": h[2], "origin": h[4:7]}
