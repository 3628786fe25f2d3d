"""Bindings to the REAL reference code, for validating the oracle and as the
"reference" CPU baseline.  TEST INFRASTRUCTURE ONLY.

Two sources of truth are reachable on a CPU-only machine:

* ``oracle/_ref/*.so`` — the reference's hash-table, kernel-map and Morton
  kernels compiled as host C++ by ``oracle/ref_build.py`` (travels with the
  repository snapshot as a built artefact; never committed);
* the reference's pure-torch Python functions (``_explicit_gemm_forward_logic``,
  ``kernel_offsets_from_size``, module init), importable from the reference tree
  once its GPU-only dependencies are stubbed.  The tree itself is only present
  on the development machine, so these are used to generate the golden fixtures
  and are skipped elsewhere.
"""
from __future__ import annotations

import ctypes
import os
import sys
import types
from unittest import mock

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
HASH_METHODS = {"fnv1a": 0, "city": 1, "murmur": 2}

_libs = {}


def have_compiled_reference() -> bool:
    return all(os.path.isfile(os.path.join(REF_DIR, n))
               for n in ("libref_hashmap.so", "libref_discrete.so", "libref_morton.so"))


def _lib(name):
    if name not in _libs:
        _libs[name] = ctypes.CDLL(os.path.join(REF_DIR, name))
    return _libs[name]


def _iptr(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_int))


class RefHashTable:
    """The reference's table: ``table_kvs [cap, 2]`` + the caller's key array,
    filled by its own insert kernel run sequentially on the host."""

    def __init__(self, keys: np.ndarray, method: str = "city", capacity: int | None = None):
        self.keys = np.ascontiguousarray(keys, dtype=np.int32)
        self.method = HASH_METHODS[method]
        n, self.key_dim = self.keys.shape
        # capacity rule of TorchHashTable.from_keys (torch_hashmap.py:218-219)
        self.capacity = max(16, 2 * n) if capacity is None else capacity
        self.table = np.empty((self.capacity, 2), dtype=np.int32)
        rc = _lib("libref_hashmap.so").ref_hash_insert(
            _iptr(self.table), _iptr(self.keys), n, self.key_dim, self.capacity, self.method)
        assert rc == 0

    def search(self, queries: np.ndarray) -> np.ndarray:
        q = np.ascontiguousarray(queries, dtype=np.int32)
        out = np.empty(len(q), dtype=np.int32)
        rc = _lib("libref_hashmap.so").ref_hash_search(
            _iptr(self.table), _iptr(self.keys), _iptr(q), _iptr(out), len(q), self.key_dim,
            self.capacity, self.method)
        assert rc == 0
        return out


def ref_kernel_map_found(in_coords, out_coords, stride, kernel_size, method="city"):
    """found[K, M] from the reference's ``kernel_map_size_4d_*`` kernel."""
    table = RefHashTable(in_coords, method)
    q = np.ascontiguousarray(np.asarray(out_coords, dtype=np.int32) * np.array([1, *stride], dtype=np.int32))
    ks = np.asarray(kernel_size, dtype=np.int32)
    K = int(np.prod(ks))
    found = np.empty((K, len(q)), dtype=np.int32)
    rc = _lib("libref_discrete.so").ref_kernel_map_size_4d(
        _iptr(table.table), _iptr(table.keys), _iptr(q), _iptr(ks), _iptr(found), len(q),
        table.capacity, K, table.method)
    assert rc == 0
    return found


def ref_compact_found(found: np.ndarray):
    """The reference's compaction: torch-side cumsum restated with NumPy
    (torch_discrete.py:103-119) + its own scatter kernel."""
    K, M = found.shape
    hit = found >= 0
    mapped = np.cumsum(hit.astype(np.int32), axis=1, dtype=np.int32) - 1
    mapped = np.maximum(mapped, -1)
    counts = (mapped.max(axis=1) + 1) if M else np.zeros(K, dtype=np.int32)
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    L = int(offsets[-1])
    in_maps = np.empty(L, dtype=np.int32)
    out_maps = np.empty(L, dtype=np.int32)
    if L:
        f = np.ascontiguousarray(found)
        mi = np.ascontiguousarray(mapped.astype(np.int32))
        rc = _lib("libref_discrete.so").ref_map_found_indices_to_maps(
            _iptr(f), _iptr(mi), _iptr(offsets), _iptr(in_maps), _iptr(out_maps), K, M)
        assert rc == 0
    return in_maps, out_maps, offsets


def ref_generate_kernel_map(in_coords, out_coords, stride, kernel_size, method="city"):
    found = ref_kernel_map_found(in_coords, out_coords, stride, kernel_size, method)
    return ref_compact_found(found)


def ref_morton20(coords_xyz: np.ndarray) -> np.ndarray:
    c = np.ascontiguousarray(coords_xyz, dtype=np.int32)
    codes = np.empty(len(c), dtype=np.int64)
    rc = _lib("libref_morton.so").ref_morton20(
        _iptr(c), len(c), codes.ctypes.data_as(ctypes.POINTER(ctypes.c_longlong)))
    assert rc == 0
    return codes


# --------------------------------------------------------------------------- reference Python (development machine only)


def reference_tree_present(root: str | None = None) -> bool:
    root = root or os.environ.get("WCN_REFERENCE_ROOT", "/root/reference")
    return os.path.isdir(os.path.join(root, "warpconvnet"))


def import_reference_python(root: str | None = None):
    """Import the reference package with cupy / warp / torch_scatter / the
    compiled ``_C`` module replaced by mocks; returns a namespace with the few
    pure-torch entry points that run on CPU tensors."""
    root = root or os.environ.get("WCN_REFERENCE_ROOT", "/root/reference")
    for name in ("cupy", "cupy.cuda", "warp", "warp.utils", "torch_scatter", "warpconvnet._C"):
        if name not in sys.modules:
            sys.modules[name] = mock.MagicMock(name=name)
    if root not in sys.path:
        sys.path.insert(0, root)
    from warpconvnet.geometry.coords.search.search_results import IntSearchResult
    from warpconvnet.geometry.coords.search.torch_discrete import kernel_offsets_from_size
    from warpconvnet.nn.functional.sparse_conv import _explicit_gemm_forward_logic
    from warpconvnet.nn.modules.sparse_conv import SpatiallySparseConv

    return types.SimpleNamespace(
        IntSearchResult=IntSearchResult,
        kernel_offsets_from_size=kernel_offsets_from_size,
        explicit_gemm_forward=_explicit_gemm_forward_logic,
        SpatiallySparseConv=SpatiallySparseConv,
    )
