"""Strided (down-sampled) output coordinates (warpconvnet/geometry/coords/ops/stride.py:17-54).

``floor(coords / stride)`` rows are made distinct through the hash table; the rows
come out in first-occurrence order, which keeps a batch-sorted input batch-sorted
and is the same on every run (the reference's order depends on insertion races
and an unstable argsort; only the set of rows is comparable with it).
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch
from torch import Tensor

from ...._native import (check, device_status, lib, ptr, query_bytes, raise_for_status, small_to_device,
                         stream_ptr)
from ....utils.ntuple import ntuple
from ..search.torch_hashmap import HashMethod
from .batch_index import offsets_from_batch_index


@torch.no_grad()
def unique_strided_rows(bcoords: Tensor, stride: Tuple[int, int, int] = (1, 1, 1),
                        hash_method: HashMethod = HashMethod.CITY, return_parent: bool = False,
                        in_offsets: Optional[Tensor] = None):
    """Distinct rows of ``floor(bcoords / [1, *stride])``.

    Returns ``(rows [M,4] int32, unique_index [M] int32, parent [N] int32 | None)``:
    ``unique_index`` are the (ascending) source rows of the first occurrences and
    ``parent[i]`` the output row input i collapsed into.  With ``in_offsets`` (the batch
    offsets of the input rows) a fourth value is returned, the CPU batch offsets of the
    output rows, obtained with the same single host synchronisation as the row count.
    """
    assert bcoords.is_cuda, f"Batched coordinates must be on cuda device, got {bcoords.device}"
    assert bcoords.dtype == torch.int32 and bcoords.ndim == 2 and bcoords.shape[1] == 4
    dev = bcoords.device
    c = bcoords.contiguous()
    n = c.shape[0]
    if n == 0:
        e = torch.empty(0, dtype=torch.int32, device=dev)
        base = (c.clone(), e, (e.clone() if return_parent else None))
        return base if in_offsets is None else base + (torch.zeros(len(in_offsets), dtype=torch.long),)
    cap = max(16, 2 * n)
    table = torch.empty(query_bytes("wcn_hash_table_bytes", cap), dtype=torch.uint8, device=dev)
    strd = (ctypes.c_int32 * 3)(*[int(s) for s in stride])
    sp = ctypes.addressof(strd)
    st = stream_ptr(dev)
    check(lib().wcn_hash_build(ptr(c), n, sp, ptr(table), cap, hash_method.value, None, ptr(device_status(dev)), st),
          "wcn_hash_build")
    ws = torch.empty(query_bytes("wcn_unique_workspace_bytes", n), dtype=torch.uint8, device=dev)
    count = torch.empty(1, dtype=torch.int64, device=dev)
    check(lib().wcn_unique_mark(ptr(c), n, sp, ptr(table), cap, hash_method.value, ptr(ws), ptr(count), st),
          "wcn_unique_mark")
    # Outputs are sized for the worst case (every row distinct) so that nothing has to be read
    # back before the rows are emitted; the one host synchronisation happens in the caller's
    # read of the count / batch offsets.
    rows = torch.empty((n, 4), dtype=torch.int32, device=dev)
    uidx = torch.full((n,), torch.iinfo(torch.int32).max, dtype=torch.int32, device=dev)
    parent = torch.empty(n, dtype=torch.int32, device=dev) if return_parent else None
    check(lib().wcn_unique_emit(ptr(c), n, sp, ptr(ws), ptr(rows), ptr(uidx), ptr(parent), st), "wcn_unique_emit")
    if in_offsets is not None:
        # first occurrences are emitted in ascending source row, so the output batch boundaries are
        # the ranks of the input boundaries among the first-occurrence rows
        # The device status word rides along in the same read: this is a point where the host waits
        # for the device anyway, so a kernel failure recorded earlier surfaces here.
        nb = len(in_offsets)
        packed = torch.empty(nb + 1, dtype=torch.int64, device=dev)
        torch.searchsorted(uidx, small_to_device(in_offsets, dev, torch.int32), out=packed[:nb])
        packed[nb:].copy_(device_status(dev))
        host = packed.cpu()
        raise_for_status(int(host[nb]), dev)
        out_offsets = host[:nb].clone()
        m = int(out_offsets[-1])
        return rows[:m], uidx[:m], parent, out_offsets
    both = torch.cat([count, device_status(dev).to(torch.int64)]).cpu()
    raise_for_status(int(both[1]), dev)
    m = int(both[0])
    return rows[:m], uidx[:m], parent


@torch.no_grad()
def strided_pyramid(bcoords: Tensor, total_strides, in_offsets: Tensor, hash_method: HashMethod = HashMethod.CITY):
    """Distinct rows of ``floor(bcoords / s)`` for SEVERAL strides ``s`` of the same rows, with ONE
    host synchronisation for all of them: ``[(rows [M_i, 4], CPU offsets [B+1]), ...]``.

    Chaining ``stride_coords`` level by level reads a row count back per level, and each read-back
    waits for the device; for small batches those waits are most of the cost of the whole
    coordinate pyramid.  Here every level is computed straight from the finest rows (more hashing,
    no dependency between levels) and the counts come back together.  Rows come out in
    first-occurrence order, which is the order the chained computation gives:
    ``floor(floor(c / 2) / 2) = floor(c / 4)``, and the first occurrence of a coarse cell among the
    finest rows is the first occurrence of its first child."""
    assert bcoords.is_cuda and bcoords.dtype == torch.int32 and bcoords.ndim == 2 and bcoords.shape[1] == 4
    dev = bcoords.device
    c = bcoords.contiguous()
    n = c.shape[0]
    nb = len(in_offsets)
    if n == 0:
        return [(c.clone(), torch.zeros(nb, dtype=torch.long)) for _ in total_strides]
    st = stream_ptr(dev)
    cap = max(16, 2 * n)
    table_bytes = query_bytes("wcn_hash_table_bytes", cap)
    ws_bytes = query_bytes("wcn_unique_workspace_bytes", n)
    offs_dev = small_to_device(in_offsets, dev, torch.int32)
    packed = torch.empty((len(total_strides), nb) if total_strides else (0, nb), dtype=torch.int64, device=dev)
    status = torch.empty(1, dtype=torch.int64, device=dev)
    outs = []
    for i, stride in enumerate(total_strides):
        strd = (ctypes.c_int32 * 3)(*[int(s) for s in stride])
        sp = ctypes.addressof(strd)
        table = torch.empty(table_bytes, dtype=torch.uint8, device=dev)
        check(lib().wcn_hash_build(ptr(c), n, sp, ptr(table), cap, hash_method.value, None, ptr(device_status(dev)), st),
              "wcn_hash_build")
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        count = torch.empty(1, dtype=torch.int64, device=dev)
        check(lib().wcn_unique_mark(ptr(c), n, sp, ptr(table), cap, hash_method.value, ptr(ws), ptr(count), st),
              "wcn_unique_mark")
        rows = torch.empty((n, 4), dtype=torch.int32, device=dev)
        uidx = torch.full((n,), torch.iinfo(torch.int32).max, dtype=torch.int32, device=dev)
        check(lib().wcn_unique_emit(ptr(c), n, sp, ptr(ws), ptr(rows), ptr(uidx), None, st), "wcn_unique_emit")
        torch.searchsorted(uidx, offs_dev, out=packed[i])
        outs.append(rows)
    status.copy_(device_status(dev))
    host = torch.cat([packed.reshape(-1), status]).cpu()  # the one synchronisation
    raise_for_status(int(host[-1]), dev)
    host = host[:-1].reshape(len(total_strides), nb)
    return [(rows[:int(host[i, -1])], host[i].clone()) for i, rows in enumerate(outs)]


@torch.no_grad()
def stride_coords(batch_indexed_coords: Tensor, stride: Tuple[int, ...], order=None,
                  in_offsets: Optional[Tensor] = None):
    """Down-sample coordinates by ``stride``; returns (coords [M,4], CPU offsets [B+1]).
    ``in_offsets`` (batch offsets of the input, when the caller has them) saves a second host
    synchronisation for the output offsets."""
    nd = batch_indexed_coords.shape[1] - 1
    assert len(stride) == nd, (f"Stride must match the number of spatial dimensions. Got {len(stride)} spatial "
                               f"dimensions for but coordinates with {nd} spatial dimensions.")
    if all(s == 1 for s in stride):
        return batch_indexed_coords, offsets_from_batch_index(batch_indexed_coords[:, 0])
    from .serialization import POINT_ORDERING, encode
    if in_offsets is not None and (order is None or order == POINT_ORDERING.RANDOM):
        rows, _, _, out_offsets = unique_strided_rows(batch_indexed_coords, ntuple(stride, ndim=nd),
                                                      in_offsets=in_offsets)
        return rows, out_offsets
    rows, _, _ = unique_strided_rows(batch_indexed_coords, ntuple(stride, ndim=nd))
    if order is not None and order != POINT_ORDERING.RANDOM:
        offsets = offsets_from_batch_index(rows[:, 0])
        perm = encode(rows[:, 1:], batch_offsets=offsets, order=order, return_perm=True).perm
        rows = rows[perm]
    return rows, offsets_from_batch_index(rows[:, 0])
