"""Kernel-map generation (warpconvnet/geometry/coords/search/torch_discrete.py:44-77, 244-466).

``generate_kernel_map`` builds the hash table on the INPUT coordinates, multiplies
the OUTPUT coordinates by the stride and, for every position of the kernel
window, looks the shifted coordinate up.  One fused kernel writes the dense
neighbour table and per-block hit counts; the compact (in_maps, out_maps,
offsets) triple is produced lazily by :class:`IntSearchResult`.
"""
from __future__ import annotations

import ctypes
from typing import Literal, Optional, Tuple

import numpy as np
import torch
from torch import Tensor

from ...._native import check, lib, ptr, query_bytes, stream_ptr
from ....utils.ntuple import ntuple
from .search_results import IntSearchResult
from .torch_hashmap import HashMethod, TorchHashTable


@torch.no_grad()
def kernel_offsets_from_size(kernel_size: Tuple[int, ...], kernel_dilation: Tuple[int, ...],
                             center_offset: Optional[Tuple[int, ...]] = None,
                             device: Optional[torch.device] = None) -> Tensor:
    """[K, D+1] int32 offsets: batch column (zero) first, last spatial axis fastest;
    centre (s-1)//2 for odd sizes, 0 for even sizes; scaled by the dilation."""
    assert len(kernel_size) == len(kernel_dilation)
    nd = len(kernel_size)
    if center_offset is None:
        center_offset = [(s - 1) // 2 if s % 2 == 1 else 0 for s in kernel_size]
    assert len(center_offset) == nd
    axes = [torch.arange(s, dtype=torch.int32) for s in kernel_size]
    grids = torch.meshgrid(*axes, indexing="ij")
    cols = [torch.zeros(int(np.prod(kernel_size)), dtype=torch.int32)]
    for d in range(nd):
        cols.append((grids[d].reshape(-1) - center_offset[d]) * kernel_dilation[d])
    return torch.stack(cols, dim=1).contiguous().to(device)


@torch.no_grad()
def _kernel_map_from_size(hashtable: TorchHashTable, batched_query_coords: Tensor,
                          kernel_sizes: Tuple[int, ...], identity_map_index: Optional[int] = None,
                          return_type: Literal["indices", "offsets"] = "offsets",
                          skip_symmetric_kernel_map: bool = False,
                          query_stride: Optional[Tuple[int, ...]] = None, num_in: Optional[int] = None,
                          self_map: bool = False, kernel_dilation: Optional[Tuple[int, ...]] = None,
                          kernel_center_offset: Optional[Tuple[int, ...]] = None, bricks=None):
    """Search every position of a ``kernel_sizes`` window around each query.

    ``return_type="indices"`` returns ``found[K, M]`` (-1 = absent), "offsets" an
    :class:`IntSearchResult`.  With ``skip_symmetric_kernel_map`` only the first
    K//2 positions are searched (torch_discrete.py:291-296).  ``self_map``: the queries are the
    rows the table was built from, in the same order (odd window, stride 1); the native call
    then probes half of the offsets and mirrors the rest when the rows are distinct.
    ``kernel_center_offset`` moves the window: position (i, j, l) probes ``x + (i - cx) * dx`` ...
    ``bricks``: a :class:`BrickTable` of the table's keys; windows up to 4 wide without dilation are
    then answered from it (same result).
    """
    dev = hashtable.device
    assert str(dev) == str(batched_query_coords.device)
    assert batched_query_coords.dtype == torch.int32
    if hashtable._table is None:
        raise RuntimeError("Input TorchHashTable must be populated before calling kernel map functions.")
    assert batched_query_coords.shape[1] == 4, "coordinates must be (batch, x, y, z) rows"
    assert len(kernel_sizes) == 3, f"kernel_size ({len(kernel_sizes)}) must match spatial dims (3)"
    K = int(np.prod(kernel_sizes))
    if skip_symmetric_kernel_map:
        assert all(k % 2 == 1 for k in kernel_sizes), f"Kernel sizes must be odd for symmetric skipping. Got {kernel_sizes}"
        K = K // 2
        if identity_map_index is not None:
            assert identity_map_index == K
    q = batched_query_coords.contiguous()
    M = q.shape[0]
    nbr = torch.empty((K, M), dtype=torch.int32, device=dev)
    ksz = (ctypes.c_int32 * 3)(*[int(k) for k in kernel_sizes])
    strd = (ctypes.c_int32 * 3)(*[int(s) for s in (query_stride or (1, 1, 1))])
    dil = (ctypes.c_int32 * 3)(*[int(d) for d in (kernel_dilation or (1, 1, 1))])
    # hit counts are only needed by the compact form; IntSearchResult makes them on demand
    ws = None
    ctr = None
    if kernel_center_offset is not None:
        assert len(kernel_center_offset) == 3
        ctr = (ctypes.c_int32 * 3)(*[int(c) for c in kernel_center_offset])
    undilated = all(int(d) == 1 for d in (kernel_dilation or (1, 1, 1)))
    if (bricks is not None and ctr is None and undilated and not skip_symmetric_kernel_map
            and all(1 <= int(k) <= 4 for k in kernel_sizes)):
        assert bricks.hashtable is hashtable, "brick table belongs to another hash table"
        check(lib().wcn_kmap_search_bricks(ptr(bricks._table), ptr(hashtable._table), hashtable.capacity,
                                           hashtable.hash_method.value, ptr(q), M, ctypes.addressof(strd),
                                           ctypes.addressof(ksz), ptr(nbr), stream_ptr(dev)), "wcn_kmap_search_bricks")
    elif (self_map and ctr is None and not skip_symmetric_kernel_map and all(k % 2 == 1 for k in kernel_sizes)
            and all(int(s) == 1 for s in (query_stride or (1, 1, 1)))):
        assert M == len(hashtable.vector_keys), "self_map needs the table's own rows as queries"
        hashtable.ensure_built()
        check(lib().wcn_kmap_search_self(ptr(hashtable._table), hashtable.capacity, hashtable.hash_method.value,
                                         ptr(q), M, ctypes.addressof(ksz), ctypes.addressof(dil), ptr(nbr),
                                         stream_ptr(dev)), "wcn_kmap_search_self")
    else:
        hashtable.ensure_built()
        check(lib().wcn_kmap_search_dilated(ptr(hashtable._table), hashtable.capacity, hashtable.hash_method.value,
                                            ptr(q), M, ctypes.addressof(strd), ctypes.addressof(ksz),
                                            ctypes.addressof(dil), ctypes.addressof(ctr) if ctr is not None else None,
                                            K, ptr(nbr), None, stream_ptr(dev)),
              "wcn_kmap_search_dilated")
    if return_type == "indices":
        return nbr
    assert return_type == "offsets"
    n_in = num_in if num_in is not None else len(hashtable.vector_keys)
    return IntSearchResult.from_neighbor_table(nbr, n_in, ws, identity_map_index)


@torch.no_grad()
def generate_kernel_map(batch_indexed_in_coords: Tensor, batch_indexed_out_coords: Tensor,
                        in_to_out_stride_ratio: Tuple[int, ...], kernel_size: Tuple[int, ...],
                        kernel_dilation: Optional[Tuple[int, ...]] = None,
                        kernel_center_offset: Optional[Tuple[int, ...]] = None,
                        method: Literal["offset", "size"] = "size",
                        hash_method: HashMethod = HashMethod.CITY,
                        skip_symmetric_kernel_map: bool = False,
                        hashtable: Optional[TorchHashTable] = None, bricks=None) -> IntSearchResult:
    """Kernel map between input and output coordinates ([N,4] / [M,4] int32).
    ``hashtable`` (an addition to the reference signature): a table already built over
    ``batch_indexed_in_coords``, to skip rebuilding it.  ``bricks`` (likewise): the
    :class:`BrickTable` of Morton-ordered input coordinates (``IntCoords.bricks``)."""
    dev = batch_indexed_in_coords.device
    assert dev == batch_indexed_out_coords.device
    assert batch_indexed_in_coords.dtype == torch.int32
    assert batch_indexed_out_coords.dtype == torch.int32
    if skip_symmetric_kernel_map:
        assert len(batch_indexed_in_coords) == len(batch_indexed_out_coords), \
            "You can only skip symmetric kernel map if the input and output coordinates are the same."
        assert all(k % 2 == 1 for k in kernel_size), "Kernel size must be odd for symmetric skipping."
    nd = batch_indexed_out_coords.shape[1] - 1
    assert len(in_to_out_stride_ratio) == nd
    stride = ntuple(in_to_out_stride_ratio, ndim=nd)

    identity_map_index = None
    is_odd = all(k % 2 == 1 for k in kernel_size)
    default_center = kernel_center_offset is None or all(
        int(c) == ((k - 1) // 2 if k % 2 == 1 else 0) for c, k in zip(kernel_center_offset, kernel_size))
    if is_odd and default_center and batch_indexed_in_coords.shape[0] == batch_indexed_out_coords.shape[0]:
        identity_map_index = int(np.prod(kernel_size)) // 2
    if skip_symmetric_kernel_map and not is_odd:
        skip_symmetric_kernel_map = False

    if method not in ("size", "offset"):
        raise ValueError(f"Invalid method: {method}. Choose 'query', 'offset', or 'size'.")
    # Both methods reduce to the window search, which takes a dilation and a window centre.  The
    # reference accepts those two only with method="offset" (torch_discrete.py:449-456).
    if method == "size":
        assert kernel_center_offset is None, \
            "Custom kernel_center_offset is not supported with method='size'. Use method='offset' instead."
    if kernel_center_offset is not None:
        assert len(kernel_center_offset) == nd and not skip_symmetric_kernel_map

    if hashtable is None or hashtable.hash_method != hash_method:
        hashtable = TorchHashTable.from_keys(batch_indexed_in_coords, hash_method=hash_method, device=dev)
    else:
        assert len(hashtable.vector_keys) == batch_indexed_in_coords.shape[0], "hashtable was built over other keys"
    if bricks is not None and bricks.hashtable is not hashtable:
        bricks = None
    return _kernel_map_from_size(hashtable, batch_indexed_out_coords, kernel_size, bricks=bricks,
                                 identity_map_index=identity_map_index, return_type="offsets",
                                 skip_symmetric_kernel_map=skip_symmetric_kernel_map, query_stride=stride,
                                 num_in=batch_indexed_in_coords.shape[0],
                                 kernel_dilation=(tuple(int(d) for d in kernel_dilation) if kernel_dilation else None),
                                 kernel_center_offset=(None if default_center else tuple(int(c) for c in kernel_center_offset)),
                                 self_map=(batch_indexed_out_coords.data_ptr() == batch_indexed_in_coords.data_ptr()
                                           and batch_indexed_out_coords.shape == batch_indexed_in_coords.shape
                                           and batch_indexed_in_coords.is_contiguous()))
