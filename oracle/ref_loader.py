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


def ref_kernel_map_found_offsets(in_coords, out_coords, stride, kernel_offsets, method="city"):
    """found[K, M] from the reference's ``kernel_map_offset_*`` kernel for an explicit offset list
    ``[K, 4]`` (what ``kernel_offsets_from_size`` returns for a dilation / custom centre)."""
    table = RefHashTable(in_coords, method)
    q = np.ascontiguousarray(np.asarray(out_coords, dtype=np.int32) * np.array([1, *stride], dtype=np.int32))
    offs = np.ascontiguousarray(kernel_offsets, dtype=np.int32)
    found = np.empty((len(offs), len(q)), dtype=np.int32)
    rc = _lib("libref_discrete.so").ref_kernel_map_offset(
        _iptr(table.table), _iptr(table.keys), _iptr(q), _iptr(offs), _iptr(found), len(q), 4, len(offs),
        table.capacity, table.method)
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
    from .ref_build import default_reference_root
    root = root or default_reference_root()
    return bool(root) and os.path.isdir(os.path.join(root, "warpconvnet"))


def import_reference_python(root: str | None = None):
    """Import the reference package with cupy / warp / torch_scatter / the
    compiled ``_C`` module replaced by mocks; returns a namespace with the few
    pure-torch entry points that run on CPU tensors."""
    from .ref_build import default_reference_root
    root = root or default_reference_root()
    if not reference_tree_present(root):
        raise RuntimeError("set WCN_REFERENCE_ROOT to the reference project's checkout")
    for name in ("cupy", "cupy.cuda", "warp", "warp.utils", "warpconvnet._C"):
        if name not in sys.modules:
            sys.modules[name] = mock.MagicMock(name=name)
    if "torch_scatter" not in sys.modules:
        # torch_scatter is not installed here.  Its ``segment_csr(src, indptr, reduce)`` reduces the
        # rows src[indptr[i]:indptr[i+1]]; PyTorch's own ``torch.segment_reduce`` does the same, so
        # the reference's ``row_reduction`` runs on top of it.
        import torch
        stand_in = types.ModuleType("torch_scatter")

        def segment_csr(src, indptr, out=None, reduce="sum"):
            return torch.segment_reduce(src, {"mul": "prod"}.get(reduce, reduce), offsets=indptr.long(), axis=0)

        stand_in.segment_csr = segment_csr
        sys.modules["torch_scatter"] = stand_in
    if root not in sys.path:
        sys.path.insert(0, root)
    from warpconvnet.geometry.coords.search.search_results import IntSearchResult
    from warpconvnet.geometry.coords.search.torch_discrete import kernel_offsets_from_size
    from warpconvnet.nn.functional.sparse_conv import _explicit_gemm_forward_logic
    from warpconvnet.nn.modules.sparse_conv import SpatiallySparseConv
    from warpconvnet.ops.reductions import row_reduction

    return types.SimpleNamespace(
        IntSearchResult=IntSearchResult,
        kernel_offsets_from_size=kernel_offsets_from_size,
        explicit_gemm_forward=_explicit_gemm_forward_logic,
        SpatiallySparseConv=SpatiallySparseConv,
        row_reduction=row_reduction,
    )


def ref_expand_coords(coords: np.ndarray, kernel_offsets: np.ndarray, kernel_batch: int, method: str = "city"):
    """The coordinate set the reference's ``expand_coords`` produces
    (warpconvnet/geometry/coords/ops/expand.py:17-64), with every hash-table search done by the
    reference's own search kernel: offsets are applied in batches of ``kernel_batch``, the
    candidates that the current table does not hold are appended, and the table is rebuilt over
    the distinct rows.  Returned in lexicographic order (the reference's row order depends on
    hash slots)."""
    base = np.ascontiguousarray(coords, dtype=np.int32)
    unique = base
    table = RefHashTable(unique, method)
    offs = np.asarray(kernel_offsets, dtype=np.int32)
    for s in range(0, len(offs), kernel_batch):
        cand = (base[None, :, :] + offs[s:s + kernel_batch, None, :]).reshape(-1, base.shape[1])
        missing = table.search(cand) < 0
        unique = np.unique(np.concatenate([unique, cand[missing]], 0), axis=0)
        table = RefHashTable(unique, method)
    return unique[np.lexsort(tuple(unique[:, d] for d in reversed(range(unique.shape[1]))))]
