"""NumPy restatement of the reference's coordinate hashing and kernel-map path.

TEST INFRASTRUCTURE ONLY (checker and timed CPU baseline); the product package
never imports this file.

Every function cites the reference lines it restates (paths relative to the
reference project root).  Results are defined by the reference only up to the
order it leaves unspecified (hash-slot placement is a race, see
``warpconvnet/csrc/hashmap_kernels.cu:191-234``), so this restatement uses exact
sort/merge arithmetic instead of mimicking the probe sequence; the probe
sequence itself is restated once, in :class:`ProbeTable`, for tiny cases.

Parity: pinned against the reference's own kernels compiled for the host
(``oracle/_ref``) in ``tests/test_oracle_pins.py`` and against the golden
vectors in ``tests/golden``.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import numpy as np

# --------------------------------------------------------------------------- offsets


def kernel_offsets_from_size(
    kernel_size: Sequence[int],
    kernel_dilation: Optional[Sequence[int]] = None,
    center_offset: Optional[Sequence[int]] = None,
) -> np.ndarray:
    """[K, D+1] int32 offsets, batch column first and zero.

    Restates ``kernel_offsets_from_size``
    (warpconvnet/geometry/coords/search/torch_discrete.py:44-77): meshgrid with
    ``indexing="ij"`` so the last spatial axis varies fastest; the centre is
    ``(s-1)//2`` for odd sizes and 0 for even sizes; offsets are scaled by the
    dilation.
    """
    kernel_size = tuple(int(s) for s in kernel_size)
    nd = len(kernel_size)
    if kernel_dilation is None:
        kernel_dilation = (1,) * nd
    if center_offset is None:
        center_offset = [(s - 1) // 2 if s % 2 == 1 else 0 for s in kernel_size]
    grids = np.meshgrid(*[np.arange(s, dtype=np.int32) for s in kernel_size], indexing="ij")
    cols = [np.zeros(int(np.prod(kernel_size)), dtype=np.int32)]
    for d in range(nd):
        cols.append(((grids[d].reshape(-1) - center_offset[d]) * kernel_dilation[d]).astype(np.int32))
    return np.stack(cols, axis=1)


# --------------------------------------------------------------------------- exact search


def _pack_rows(rows_list):
    """Map int32 [*, D] row arrays to int64 scalars with one shared mixed radix.
    Columns whose raw range would overflow are first replaced by their dense rank."""
    nonempty = [r for r in rows_list if len(r)]
    mins = np.min([r.min(axis=0) for r in nonempty], axis=0).astype(np.int64)
    maxs = np.max([r.max(axis=0) for r in nonempty], axis=0).astype(np.int64)
    span = maxs - mins + 1
    total = 1
    for s in span:
        total *= int(s)
    cols = [[r[:, d].astype(np.int64) - mins[d] for d in range(r.shape[1])] for r in rows_list]
    if total >= 2**62:
        for d in range(len(span)):
            allv = np.concatenate([c[d] for c in cols])
            uniq, inv = np.unique(allv, return_inverse=True)
            span[d] = len(uniq)
            pos = 0
            for c in cols:
                c[d] = inv[pos:pos + len(c[d])].astype(np.int64)
                pos += len(c[d])
        total = 1
        for s in span:
            total *= int(s)
        assert total < 2**62, "too many distinct coordinate values for the oracle's int64 packing"
    packed = []
    for c, r in zip(cols, rows_list):
        acc = np.zeros(len(r), dtype=np.int64)
        for d in range(r.shape[1]):
            acc = acc * span[d] + c[d]
        packed.append(acc)
    return packed


def hash_search(keys: np.ndarray, queries: np.ndarray) -> np.ndarray:
    """Row index of each query in ``keys`` or -1.

    Restates the observable result of ``TorchHashTable.search``
    (warpconvnet/geometry/coords/search/torch_hashmap.py:225-301) backed by
    ``search_hash_table`` (warpconvnet/csrc/hashmap_kernels.cu:133-177): the
    index into the inserted key array, -1 when absent.  With duplicate keys the
    reference returns whichever duplicate won a probe slot; here the smallest
    index is returned (callers that need the reference's freedom compare sets).
    """
    keys = np.ascontiguousarray(keys, dtype=np.int32)
    queries = np.ascontiguousarray(queries, dtype=np.int32)
    out = np.full(len(queries), -1, dtype=np.int32)
    if len(keys) == 0 or len(queries) == 0:
        return out
    pk, pq = _pack_rows([keys, queries])
    order = np.argsort(pk, kind="stable")
    sk = pk[order]
    pos = np.searchsorted(sk, pq, side="left")
    pos_c = np.minimum(pos, len(sk) - 1)
    hit = sk[pos_c] == pq
    out[hit] = order[pos_c[hit]].astype(np.int32)
    return out


# --------------------------------------------------------------------------- kernel map


def identity_map_index(kernel_size: Sequence[int], n_in: int, n_out: int) -> Optional[int]:
    """``K//2`` iff every kernel size is odd and the two coordinate arrays have
    the same length (warpconvnet/geometry/coords/search/torch_discrete.py:418-425)."""
    if all(int(k) % 2 == 1 for k in kernel_size) and n_in == n_out:
        return int(np.prod(kernel_size)) // 2
    return None


def kernel_map_found(
    in_coords: np.ndarray, out_coords: np.ndarray, stride: Sequence[int], kernel_size: Sequence[int],
    kernel_dilation: Optional[Sequence[int]] = None, center_offset: Optional[Sequence[int]] = None
) -> np.ndarray:
    """found[K, M]: input row matching ``out*stride + offset[k]`` or -1 (offsets scaled by the
    dilation and shifted by a custom window centre, torch_discrete.py:60-77).

    Restates ``kernel_map_size_4d_templated``
    (warpconvnet/csrc/discrete_kernels.cu:264-334) and, for dilated or re-centred windows,
    ``kernel_map_offset_templated`` (discrete_kernels.cu:129-180) with the stride product of
    ``generate_kernel_map`` (torch_discrete.py:406-416).
    """
    in_coords = np.ascontiguousarray(in_coords, dtype=np.int32)
    out_coords = np.ascontiguousarray(out_coords, dtype=np.int32)
    offs = kernel_offsets_from_size(kernel_size, kernel_dilation, center_offset)
    K, M = len(offs), len(out_coords)
    svec = np.array([1, *stride], dtype=np.int32)
    q0 = out_coords * svec
    found = np.empty((K, M), dtype=np.int32)
    if M == 0:
        return found
    allq = (q0[None, :, :] + offs[:, None, :]).reshape(K * M, -1)
    found[:] = hash_search(in_coords, allq).reshape(K, M)
    return found


def compact_found(found: np.ndarray) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """(in_maps[L], out_maps[L], offsets[K+1]) from found[K, M].

    Restates ``_kernel_map_search_to_result`` (torch_discrete.py:80-157) and
    ``map_found_indices_to_maps_kernel`` (discrete_kernels.cu:183-213): within
    one offset the pairs are in ascending output index.
    """
    K, M = found.shape
    hit = found >= 0
    counts = hit.sum(axis=1).astype(np.int32)
    offsets = np.zeros(K + 1, dtype=np.int32)
    np.cumsum(counts, out=offsets[1:])
    kk, mm = np.nonzero(hit)  # row-major: k ascending, then m ascending
    return found[kk, mm].astype(np.int32), mm.astype(np.int32), offsets


def generate_kernel_map(in_coords, out_coords, stride, kernel_size, kernel_dilation=None):
    """Full map as the reference's ``generate_kernel_map`` (torch_discrete.py:365-466,
    method="size") returns it: in_maps, out_maps, offsets, identity_map_index."""
    found = kernel_map_found(in_coords, out_coords, stride, kernel_size, kernel_dilation)
    in_maps, out_maps, offsets = compact_found(found)
    return in_maps, out_maps, offsets, identity_map_index(kernel_size, len(in_coords), len(out_coords))


def transposed_kernel_map(in_coords_coarse, out_coords_fine, stride, kernel_size):
    """Map of a transposed convolution (coarse -> fine).

    Restates nn/functional/sparse_conv.py:1945-1958: the forward map is built
    with the FINE coordinates in the table and the COARSE coordinates times the
    stride as queries, then in/out are swapped; the identity index is dropped.
    """
    fin, fout, offsets, _ = generate_kernel_map(out_coords_fine, in_coords_coarse, stride, kernel_size)
    return fout, fin, offsets, None


def expand_coords(coords: np.ndarray, kernel_size: Sequence[int], kernel_dilation: Optional[Sequence[int]] = None):
    """Set of coordinates a kernel window reaches from ``coords`` (the reference's ``expand_coords``,
    warpconvnet/geometry/coords/ops/expand.py:17-64, whose row order depends on hash slots): returned
    in lexicographic order with its batch offsets."""
    coords = np.ascontiguousarray(coords, dtype=np.int32)
    offs = kernel_offsets_from_size(kernel_size, kernel_dilation)
    cand = (coords[None, :, :] + offs[:, None, :]).reshape(-1, coords.shape[1])
    out = canonical_coords(np.unique(np.concatenate([coords, cand], axis=0), axis=0))
    nb = int(out[:, 0].max()) + 1 if len(out) else 0
    counts = np.bincount(out[:, 0], minlength=nb)
    return out, np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)


# --------------------------------------------------------------------------- stride


def stride_coords(coords: np.ndarray, stride: Sequence[int]) -> Tuple[np.ndarray, np.ndarray]:
    """Distinct rows of ``floor(coords / [1, *stride])`` and their batch offsets.

    Restates ``stride_coords`` (warpconvnet/geometry/coords/ops/stride.py:17-54)
    with ``unique_hashmap`` (warpconvnet/utils/unique.py:125-144).  The reference
    divides in floating point and floors, which equals integer floor division
    while |coord| < 2**24; its output row ORDER within a batch depends on insert
    races and an unstable argsort, so only the set is defined.  This function
    returns the rows in first-occurrence order (which is batch-sorted when the
    input is), the order the product also produces.
    """
    coords = np.ascontiguousarray(coords, dtype=np.int32)
    svec = np.array([1, *stride], dtype=np.int32)
    q = np.floor_divide(coords, svec).astype(np.int32)
    if len(q) == 0:
        return q, np.zeros(1, dtype=np.int64)
    (pq,) = _pack_rows([q])
    _, first = np.unique(pq, return_index=True)
    first.sort()
    out = q[first]
    nb = int(out[:, 0].max()) + 1
    counts = np.bincount(out[:, 0], minlength=nb)
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)
    return out, offsets


# --------------------------------------------------------------------------- morton


def _part1by2(n: np.ndarray) -> np.ndarray:
    n = n.astype(np.uint64)
    n = (n ^ (n << np.uint64(32))) & np.uint64(0xFFFF00000000FFFF)
    n = (n ^ (n << np.uint64(16))) & np.uint64(0x00FF0000FF0000FF)
    n = (n ^ (n << np.uint64(8))) & np.uint64(0xF00F00F00F00F00F)
    n = (n ^ (n << np.uint64(4))) & np.uint64(0x30C30C30C30C30C3)
    n = (n ^ (n << np.uint64(2))) & np.uint64(0x9249249249249249)
    return n


def morton_code(coords_xyz: np.ndarray, subtract_min: bool = True) -> np.ndarray:
    """int64 Morton code, x in bit 0, y in bit 1, z in bit 2.

    Restates ``morton_code_20bit_device`` (warpconvnet/csrc/morton_code.cu:15-22,49-56)
    after the per-axis minimum subtraction of ``morton_code``
    (warpconvnet/geometry/coords/ops/serialization.py:224-225).
    """
    c = np.ascontiguousarray(coords_xyz, dtype=np.int64)
    if len(c) == 0:
        return np.zeros(0, dtype=np.int64)
    if subtract_min:
        c = c - c.min(axis=0)
    code = (_part1by2(c[:, 2]) << np.uint64(2)) | (_part1by2(c[:, 1]) << np.uint64(1)) | _part1by2(c[:, 0])
    return code.astype(np.int64)


# --------------------------------------------------------------------------- canonical forms


def lex_rank(coords: np.ndarray) -> np.ndarray:
    """rank[i] = position of row i in lexicographic (b, x, y, z) order."""
    order = np.lexsort(tuple(coords[:, d] for d in reversed(range(coords.shape[1]))))
    rank = np.empty(len(coords), dtype=np.int64)
    rank[order] = np.arange(len(coords))
    return rank


def canonical_kernel_map(in_maps, out_maps, offsets, in_coords=None, out_coords=None):
    """Canonical form used for "bit-exact after canonical sorting".

    Indices are mapped through the lexicographic rank of their own coordinate
    array (when given); within every offset the pairs are sorted by (out, in).
    Returns (in', out', offsets) as int64/int64/int64 arrays.
    """
    in_maps = np.asarray(in_maps, dtype=np.int64)
    out_maps = np.asarray(out_maps, dtype=np.int64)
    offsets = np.asarray(offsets, dtype=np.int64)
    if in_coords is not None:
        in_maps = lex_rank(np.asarray(in_coords))[in_maps]
    if out_coords is not None:
        out_maps = lex_rank(np.asarray(out_coords))[out_maps]
    ci, co = in_maps.copy(), out_maps.copy()
    for k in range(len(offsets) - 1):
        s, e = offsets[k], offsets[k + 1]
        o = np.lexsort((in_maps[s:e], out_maps[s:e]))
        ci[s:e] = in_maps[s:e][o]
        co[s:e] = out_maps[s:e][o]
    return ci, co, offsets



def tile_order_window(num_rows: int) -> int:
    """Window of the product's tile order: 4096 rows for tables of at most 4096 rows, else 16384."""
    return 4096 if num_rows <= 4096 else 16384


def tile_order_key(found: np.ndarray) -> np.ndarray:
    """Sort key of the product's tile order: the presence mask ``sum_k (found[k, m] >= 0) << pos(k)``.
    For a 3x3x3 window (27 offsets) ``pos`` puts the centre offset in bit 0, then the 6 face, the 12 edge
    and the 8 corner offsets, each class in offset order; otherwise ``pos(k) = k``."""
    found = np.asarray(found)
    K, M = found.shape
    if K == 27:
        cls = [(k // 9 != 1) + ((k // 3) % 3 != 1) + (k % 3 != 1) for k in range(27)]
        order = sorted(range(27), key=lambda k: (cls[k], k))
        pos = {k: i for i, k in enumerate(order)}
    else:
        pos = {k: k for k in range(K)}
    key = np.zeros(M, dtype=np.uint64)
    for k in range(K):
        key |= (found[k] >= 0).astype(np.uint64) << np.uint64(pos[k])
    return key


def tile_order(found: np.ndarray, window: int = 0) -> Tuple[np.ndarray, np.ndarray]:
    """Row order used by the product's tiled neighbour table (its own layout, no reference
    counterpart): inside each window of consecutive output rows (``tile_order_window``), rows sorted by
    ``tile_order_key``, ties by row.  Returns ``(out_rows[M], found[:, out_rows])``."""
    found = np.asarray(found)
    K, M = found.shape
    window = window or tile_order_window(M)
    key = tile_order_key(found)
    rows = np.arange(M, dtype=np.int64)
    for s in range(0, M, window):
        e = min(M, s + window)
        rows[s:e] = s + np.argsort(key[s:e], kind="stable")
    return rows.astype(np.int32), found[:, rows]


def canonical_coords(coords: np.ndarray) -> np.ndarray:
    """Rows sorted lexicographically by (b, x, y, z)."""
    coords = np.asarray(coords)
    order = np.lexsort(tuple(coords[:, d] for d in reversed(range(coords.shape[1]))))
    return coords[order]


# --------------------------------------------------------------------------- probe-sequence restatement (tiny cases)

_M32 = 0xFFFFFFFF


def _city_mix(h: int, k: int) -> int:
    # warpconvnet/csrc/hashmap_kernels.cu:38-46
    h = (h + (k * 0x9E3779B9 & _M32)) & _M32
    h ^= h >> 16
    h = (h * 0x85EBCA6B) & _M32
    h ^= h >> 13
    h = (h * 0xC2B2AE35) & _M32
    h ^= h >> 16
    return h


def _fnv1a_mix(h: int, k: int) -> int:
    # warpconvnet/csrc/hashmap_kernels.cu:32-36
    return ((h ^ k) * 16777619) & _M32


def _murmur_mix(h: int, k: int) -> int:
    # warpconvnet/csrc/hashmap_kernels.cu:8-20
    k = (k * 0xCC9E2D51) & _M32
    k = ((k << 15) | (k >> 17)) & _M32
    k = (k * 0x1B873593) & _M32
    h ^= k
    h = ((h << 13) | (h >> 19)) & _M32
    return (h * 5 + 0xE6546B64) & _M32


def reference_slot(key: Sequence[int], capacity: int, method: str = "city") -> int:
    """Home slot of a key (warpconvnet/csrc/hashmap_kernels.cu:85-118): 32-bit
    mix folded over the key ints, reinterpreted as signed, C-style ``%`` with the
    ``+cap) % cap`` fix-up."""
    ks = [int(k) & _M32 for k in key]
    if method == "city":
        h = 0
        for k in ks:
            h = _city_mix(h, k)
    elif method == "fnv1a":
        h = 2166136261
        for k in ks:
            h = _fnv1a_mix(h, k)
    elif method == "murmur":
        h = 0x9747B28C
        for k in ks:
            h = _murmur_mix(h, k)
        h ^= len(ks) * 4
        h ^= h >> 16
        h = (h * 0x85EBCA6B) & _M32
        h ^= h >> 13
        h = (h * 0xC2B2AE35) & _M32
        h ^= h >> 16
    else:
        raise ValueError(method)
    signed = h - (1 << 32) if h & 0x80000000 else h
    rem = abs(signed) % capacity
    rem = -rem if signed < 0 else rem  # C remainder truncates toward zero
    return (rem + capacity) % capacity


class ProbeTable:
    """Pure-Python open-addressing table with the reference's probe sequence
    (sequential insertion order).  Restates ``insert_kernel_templated`` and
    ``search_hash_table`` (warpconvnet/csrc/hashmap_kernels.cu:133-234); capacity
    rule ``max(16, 2N)`` from torch_hashmap.py:218-219.  For tiny cases only."""

    def __init__(self, keys: np.ndarray, method: str = "city"):
        self.keys = np.asarray(keys, dtype=np.int32)
        self.method = method
        self.capacity = max(16, 2 * len(self.keys))
        self.marker = [-1] * self.capacity
        self.value = [-1] * self.capacity
        for idx, key in enumerate(self.keys):
            slot = reference_slot(key, self.capacity, method)
            for _ in range(self.capacity):
                if self.marker[slot] == -1:
                    self.marker[slot] = slot
                    self.value[slot] = idx
                    break
                slot = (slot + 1) % self.capacity

    def search(self, queries: np.ndarray) -> np.ndarray:
        out = np.full(len(queries), -1, dtype=np.int32)
        for qi, q in enumerate(np.asarray(queries, dtype=np.int32)):
            slot = reference_slot(q, self.capacity, self.method)
            for _ in range(self.capacity):
                if self.marker[slot] == -1:
                    break
                v = self.value[slot]
                if v != -1 and np.array_equal(self.keys[v], q):
                    out[qi] = v
                    break
                slot = (slot + 1) % self.capacity
        return out
