"""GPU open-addressing hash table of int32 (batch, x, y, z) keys.

Surface of the reference's ``TorchHashTable``
(warpconvnet/geometry/coords/search/torch_hashmap.py:35-425): ``from_keys``,
``insert``, ``search``, ``unique_index``, ``vector_keys``, ``capacity``,
``key_dim``, ``to_dict`` / ``from_dict``.  The table itself is this library's own
layout (16-byte key + value per slot, see ``include/wcn_b200.h``); slot placement
is not part of the contract, lookups are.  Duplicate keys resolve to the smallest
row index (the reference: whichever duplicate won a race).
"""
from __future__ import annotations

import enum
from typing import Union

import numpy as np
import torch
from torch import Tensor

from ...._native import (check, lib, ptr, query_bytes, require_cuda, stream_ptr, device_status)


class HashMethod(enum.Enum):
    FNV1A = 0
    CITY = 1
    MURMUR = 2

    def kernel_suffix(self) -> str:
        return self.name.lower()


def _as_int32_keys(keys: Tensor, what: str) -> Tensor:
    if keys.dtype != torch.int32:
        if keys.dtype == torch.int64:
            keys = keys.to(torch.int32)
        else:
            raise TypeError(f"Input {what} must have dtype torch.int32, got {keys.dtype}")
    return keys.contiguous()


class TorchHashTable:
    def __init__(self, capacity: int, hash_method: HashMethod = HashMethod.CITY,
                 device: Union[str, torch.device] = "cuda"):
        if not isinstance(hash_method, HashMethod):
            raise TypeError(f"hash_method must be a HashMethod enum member, got {type(hash_method)}")
        assert capacity > 0
        self._capacity = int(capacity)
        self._hash_method_enum = hash_method
        self._device = torch.device(device)
        self._table = None        # uint8 buffer of wcn_hash_table_bytes(capacity)
        self._vector_keys = None  # [N, 4] int32 as inserted
        self._key_dim = -1
        self._standby = False  # True: built only if a brick table was unusable (decided on the device)

    # -- properties
    @property
    def capacity(self) -> int:
        return self._capacity

    @property
    def hash_method(self) -> HashMethod:
        return self._hash_method_enum

    @property
    def device(self) -> torch.device:
        return self._table.device if self._table is not None else self._device

    @property
    def key_dim(self) -> int:
        return self._key_dim

    @property
    def vector_keys(self) -> Tensor:
        if self._vector_keys is None:
            raise RuntimeError("Hash table has not been populated. Call insert() or from_keys() first.")
        return self._vector_keys

    # -- build
    def insert(self, vec_keys: Tensor, threads_per_block: int = 256, standby_for=None):
        """``standby_for`` (an addition to the reference signature): a :class:`BrickTable` of the same
        keys, built earlier on this stream.  The insert kernels then return at once when that table is
        usable, and this table is filled for real the first time something probes it directly
        (:meth:`search`, a dilated or custom-centred kernel map); a kernel map through the brick
        table needs it only when the brick table is unusable, which is exactly when it was filled."""
        if not isinstance(vec_keys, Tensor):
            raise TypeError(f"Input vec_keys must be a PyTorch Tensor, got {type(vec_keys)}")
        if not vec_keys.is_cuda:
            raise ValueError(f"Input vec_keys must be on a CUDA device, got {vec_keys.device}")
        if vec_keys.ndim != 2:
            raise ValueError(f"Input vec_keys must be 2D, got {vec_keys.ndim} dimensions")
        if self._table is not None and vec_keys.device != self.device:
            vec_keys = vec_keys.to(self.device)
        vec_keys = _as_int32_keys(vec_keys, "vec_keys")
        num_keys, key_dim = vec_keys.shape
        if key_dim != 4:
            raise ValueError(f"keys must be (batch, x, y, z) rows; got key_dim={key_dim}")
        assert num_keys <= self._capacity / 2, (
            f"Number of keys {num_keys} exceeds half the capacity {self._capacity}")
        dev = vec_keys.device
        self._key_dim = key_dim
        self._vector_keys = vec_keys
        nbytes = query_bytes("wcn_hash_table_bytes", self._capacity)
        self._table = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        self._standby = standby_for is not None  # (no reference to the brick table: it refers to this one)
        skip_if = lib().wcn_brick_usable_flag(ptr(standby_for._table)) if standby_for is not None else None
        check(lib().wcn_hash_build(ptr(vec_keys), num_keys, None, ptr(self._table), self._capacity,
                                   self._hash_method_enum.value, skip_if, ptr(device_status(dev)), stream_ptr(dev)),
              "wcn_hash_build")

    def ensure_built(self):
        """Fill a table whose build was left to the device's decision (``standby_for``).  Enqueues the
        unconditional build once; no host synchronisation."""
        if self._standby:
            self._standby = False
            dev = self._table.device
            check(lib().wcn_hash_build(ptr(self._vector_keys), len(self._vector_keys), None, ptr(self._table),
                                       self._capacity, self._hash_method_enum.value, None, ptr(device_status(dev)),
                                       stream_ptr(dev)), "wcn_hash_build")

    @classmethod
    def from_keys(cls, vec_keys: Tensor, hash_method: HashMethod = HashMethod.CITY,
                  device: Union[str, torch.device, None] = None, standby_for=None):
        if not isinstance(vec_keys, Tensor):
            vec_keys = torch.as_tensor(vec_keys)
        if device is not None and vec_keys.device != torch.device(device):
            vec_keys = vec_keys.to(device)
        if vec_keys.ndim != 2:
            raise ValueError(f"Input vec_keys for from_keys must be 2D, got {vec_keys.ndim} dimensions")
        # capacity rule of the reference (torch_hashmap.py:218-219)
        obj = cls(capacity=max(16, int(len(vec_keys) * 2)), hash_method=hash_method, device=vec_keys.device)
        obj.insert(vec_keys, standby_for=standby_for)
        return obj

    # -- query
    def search(self, search_keys: Union[Tensor, np.ndarray], threads_per_block: int = 256) -> Tensor:
        if self._table is None:
            raise RuntimeError("Hash table has not been populated. Call insert() or from_keys() first.")
        dev = self.device
        if not isinstance(search_keys, Tensor):
            try:
                search_keys = torch.as_tensor(search_keys, device=dev)
            except Exception as e:
                raise TypeError(f"Could not convert input search_keys to a Torch Tensor on device {dev}: {e}")
        if search_keys.device != dev:
            search_keys = search_keys.to(dev)
        if search_keys.ndim != 2:
            raise ValueError(f"Input search_keys must be 2D, got {search_keys.ndim} dimensions")
        if search_keys.shape[1] != self._key_dim:
            raise ValueError(f"Search keys dimension ({search_keys.shape[1]}) must match "
                             f"inserted keys dimension ({self._key_dim})")
        search_keys = _as_int32_keys(search_keys, "search_keys")
        self.ensure_built()
        results = torch.empty(len(search_keys), dtype=torch.int32, device=dev)
        check(lib().wcn_hash_search(ptr(self._table), self._capacity, self._hash_method_enum.value,
                                    ptr(search_keys), len(search_keys), ptr(results), stream_ptr(dev)),
              "wcn_hash_search")
        return results

    @property
    def unique_index(self) -> Tensor:
        """Sorted row indices, one per distinct key (its first occurrence)."""
        indices = self.search(self.vector_keys)
        return torch.unique(indices[indices != -1])

    @property
    def unique_vector_keys(self) -> Tensor:
        return self.vector_keys[self.unique_index.long()]

    # -- (de)serialisation: the key array and parameters are enough to rebuild
    def to_dict(self):
        return {"vector_keys": self.vector_keys.cpu(), "capacity": self._capacity,
                "hash_method": self._hash_method_enum.value, "key_dim": self._key_dim}

    @classmethod
    def from_dict(cls, data, device: Union[str, torch.device] = "cuda"):
        obj = cls(capacity=data["capacity"], hash_method=HashMethod(data["hash_method"]), device=device)
        obj.insert(data["vector_keys"].to(device))
        return obj
