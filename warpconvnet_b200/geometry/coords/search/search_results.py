"""``IntSearchResult``: the kernel map of a sparse convolution.

Public fields as in the reference (warpconvnet/geometry/coords/search/search_results.py:54-174):
``in_maps[L]``, ``out_maps[L]`` (int32, device), ``offsets[K+1]`` (CPU) and
``identity_map_index``; ``result[k]`` slices one kernel offset.

Two interchangeable internal forms are kept, each built from the other on first
use: the compact triple above, and the dense neighbour table ``nbr[K, M]``
(input row of output row m at offset k, or -1) that the output-stationary
convolution kernels read.  Maps produced by ``generate_kernel_map`` start dense,
so a network forward that only runs the implicit-GEMM kernels never compacts and
never synchronises with the host.
"""
from __future__ import annotations

from typing import List, Literal, Optional, Tuple

import torch
from torch import Tensor

from ...._native import check, device_status, lib, ptr, query_bytes, raise_for_status, small_to_device, stream_ptr


class IntSearchResult:
    identity_map_index: Optional[int]

    def __init__(self, in_maps: Tensor, out_maps: Tensor, offsets: Tensor,
                 identity_map_index: Optional[int] = None):
        assert len(in_maps) == len(out_maps) == int(offsets[-1].item())
        self._in_maps = in_maps
        self._out_maps = out_maps
        self._offsets = offsets.cpu()
        self.identity_map_index = identity_map_index
        self._nbr = None          # [K, M] int32
        self._num_out = None
        self._num_in = None
        self._workspace = None    # per-block hit counts of the dense form
        self._forward = None
        self._tiled = None        # (nbr_tiled [K, M], out_rows [M]) of tiled_neighbor_table
        self._num_offsets = len(self._offsets) - 1

    # -- dense construction (used by generate_kernel_map)
    @classmethod
    def from_neighbor_table(cls, nbr: Tensor, num_in: int, workspace: Optional[Tensor] = None,
                            identity_map_index: Optional[int] = None) -> "IntSearchResult":
        self = cls.__new__(cls)
        self._in_maps = self._out_maps = self._offsets = None
        self.identity_map_index = identity_map_index
        self._nbr = nbr
        self._num_offsets, self._num_out = int(nbr.shape[0]), int(nbr.shape[1])
        self._num_in = int(num_in)
        self._workspace = workspace
        self._forward = None      # set on transposed views: the map this one was swapped from
        self._tiled = None
        return self

    def _compact(self):
        if self._offsets is not None:
            return
        if self._workspace is None and self._forward is not None:
            # transposed view: the compact form is the forward map's with in/out exchanged
            fwd = self._forward
            self._in_maps, self._out_maps, self._offsets = fwd.out_maps, fwd.in_maps, fwd.offsets
            return
        nbr, K, M = self._nbr, self._num_offsets, self._num_out
        dev = nbr.device
        ws = self._workspace
        if ws is None:  # searched without hit counts: count now
            ws = torch.empty(query_bytes("wcn_kmap_workspace_bytes", M, K), dtype=torch.uint8, device=dev)
            check(lib().wcn_kmap_count(ptr(nbr), M, K, ptr(ws), stream_ptr(dev)), "wcn_kmap_count")
        offsets = torch.empty(K + 1, dtype=torch.int32, device=dev)
        check(lib().wcn_kmap_scan(ptr(ws), M, K, ptr(offsets), stream_ptr(dev)), "wcn_kmap_scan")
        # the one host synchronisation of a compact map; the device status word is read with it
        both = torch.cat([offsets, device_status(dev)]).cpu()
        raise_for_status(int(both[-1]), dev)
        offsets_cpu = both[:-1].clone()
        L = int(offsets_cpu[-1])
        in_maps = torch.empty(L, dtype=torch.int32, device=dev)
        out_maps = torch.empty(L, dtype=torch.int32, device=dev)
        check(lib().wcn_kmap_compact(ptr(nbr), M, K, ptr(ws), ptr(offsets), ptr(in_maps), ptr(out_maps),
                                     stream_ptr(dev)), "wcn_kmap_compact")
        self._in_maps, self._out_maps, self._offsets = in_maps, out_maps, offsets_cpu
        self._workspace = None  # counts were scanned in place; not reusable

    @property
    def in_maps(self) -> Tensor:
        self._compact()
        return self._in_maps

    @property
    def out_maps(self) -> Tensor:
        self._compact()
        return self._out_maps

    @property
    def offsets(self) -> Tensor:
        self._compact()
        return self._offsets

    def neighbor_table(self, num_out: int) -> Tensor:
        """``nbr[K, num_out]`` int32 on the maps' device."""
        if self._nbr is not None:
            assert self._num_out == num_out, f"kernel map was built for {self._num_out} outputs, got {num_out}"
            return self._nbr
        if self._in_maps is None:  # a transposed view whose table has not been asked for yet
            fwd = self._forward
            assert self._num_out == num_out, f"kernel map was built for {self._num_out} outputs, got {num_out}"
            dev = fwd._nbr.device
            nbr_t = torch.empty((self._num_offsets, num_out), dtype=torch.int32, device=dev)
            check(lib().wcn_nbr_transpose(ptr(fwd._nbr), fwd._num_offsets, fwd._num_out, num_out, ptr(nbr_t),
                                          stream_ptr(dev)), "wcn_nbr_transpose")
            self._nbr = nbr_t
            return nbr_t
        dev = self._in_maps.device
        K = self._num_offsets
        nbr = torch.empty((K, num_out), dtype=torch.int32, device=dev)
        offs = small_to_device(self._offsets, dev, torch.int32)
        check(lib().wcn_nbr_from_maps(ptr(self._in_maps.contiguous()), ptr(self._out_maps.contiguous()), ptr(offs),
                                      K, len(self._in_maps), num_out, ptr(nbr), stream_ptr(dev)),
              "wcn_nbr_from_maps")
        self._nbr, self._num_out = nbr, num_out
        return nbr

    def tiled_neighbor_table(self, num_out: int) -> Tuple[Tensor, Tensor]:
        """``(nbr_tiled[K, num_out], out_rows[num_out])``: the neighbour table with the output
        rows of every 16384-row window grouped by which offsets have a neighbour, and the output
        row each slot stands for.  A 128-row tile of it has far fewer offsets with any
        neighbour than a tile of consecutive rows (12 instead of 18.5 of 27 on a 2 cm room
        scan), and the convolution kernels skip the empty ones.  Built once per map, so every
        layer that shares the map shares the order."""
        if self._tiled is None:
            nbr = self.neighbor_table(num_out)
            dev = nbr.device
            tiled = torch.empty_like(nbr)
            rows = torch.empty(num_out, dtype=torch.int32, device=dev)
            check(lib().wcn_kmap_tile_order(ptr(nbr), num_out, self._num_offsets, ptr(rows), ptr(tiled),
                                            stream_ptr(dev)), "wcn_kmap_tile_order")
            self._tiled = (tiled, rows)
        assert self._tiled[0].shape[1] == num_out
        return self._tiled

    def tile_masks(self, num_out: int, tiled: bool = False) -> Tensor:
        """Per 128 consecutive rows of the neighbour table (the tiled one with ``tiled``), the set of
        offsets (bit k) that have any neighbour there; ``int32 [ceil(num_out / 128)]``, built once."""
        store = self.__dict__.setdefault("_tile_masks", {})
        if tiled not in store:
            nbr = self.tiled_neighbor_table(num_out)[0] if tiled else self.neighbor_table(num_out)
            masks = torch.empty((num_out + 127) // 128, dtype=torch.int32, device=nbr.device)
            check(lib().wcn_kmap_tile_masks(ptr(nbr), num_out, self._num_offsets, ptr(masks), stream_ptr(nbr.device)),
                  "wcn_kmap_tile_masks")
            store[tiled] = masks
        return store[tiled]

    def swapped(self, num_in: Optional[int] = None) -> "IntSearchResult":
        """The map with inputs and outputs exchanged (transposed convolution,
        warpconvnet/nn/functional/sparse_conv.py:1934-1938)."""
        if self._forward is not None and self._in_maps is None and (num_in is None or int(num_in) == self._forward._num_out):
            return self._forward  # exchanging a transposed view back gives the map it came from
        if self._offsets is None and self._nbr is not None and (num_in or self._num_in) is not None:
            # Both forms of the view come from this map when first asked for: the compact one by exchanging
            # in and out, the dense one by transposing the table (a layer that runs from the input side,
            # sparse_conv_rows_fused, needs neither: it reads this map's own table).
            out = IntSearchResult.__new__(IntSearchResult)
            out._in_maps = out._out_maps = out._offsets = None
            out.identity_map_index = None
            out._nbr = None
            out._num_offsets = self._num_offsets
            out._num_out = int(num_in if num_in is not None else self._num_in)
            out._num_in = self._num_out
            out._workspace = None
            out._forward = self
            out._tiled = None
            return out
        return IntSearchResult(self.out_maps, self.in_maps, self.offsets)

    # -- reference API
    @torch.no_grad()
    def __getitem__(self, idx: int) -> Tuple[Tensor, Tensor]:
        start, end = int(self.offsets[idx]), int(self.offsets[idx + 1])
        return self.in_maps[start:end], self.out_maps[start:end]

    @torch.no_grad()
    def get_batch(self, start_idx: int, end_idx: int, out_format: Literal["list", "tensor"] = "list"):
        ins = [self[i][0] for i in range(start_idx, end_idx)]
        outs = [self[i][1] for i in range(start_idx, end_idx)]
        if out_format == "list":
            return ins, outs
        if out_format != "tensor":
            raise ValueError(f"Invalid output format: {out_format}")
        width = max(len(x) for x in ins)
        it = torch.full((len(ins), width), -1, dtype=torch.int64, device=self.device)
        ot = torch.full((len(ins), width), -1, dtype=torch.int64, device=self.device)
        for i, (a, b) in enumerate(zip(ins, outs)):
            it[i, :len(a)] = a
            ot[i, :len(b)] = b
        return it, ot

    def __len__(self):
        return self._num_offsets

    def __iter__(self):
        for i in range(len(self)):
            yield self[i]

    def __repr__(self):
        return f"{self.__class__.__name__}(len={len(self)}, iden_map={self.identity_map_index})"

    def numel(self, i: int) -> int:
        return int(self.offsets[i + 1] - self.offsets[i])

    @torch.no_grad()
    def to_csr(self):
        out_sorted, order = torch.sort(self.out_maps)
        uniq, counts = torch.unique(out_sorted, return_counts=True, sorted=True)
        offsets = torch.cat([torch.zeros(1, dtype=torch.int32), torch.cumsum(counts.cpu(), dim=0)], dim=0)
        return self.in_maps[order], uniq, offsets

    def clone(self):
        return IntSearchResult(self.in_maps.clone(), self.out_maps.clone(), self.offsets.clone(),
                               self.identity_map_index)

    @property
    def device(self):
        if self._nbr is not None:
            return self._nbr.device
        return self._in_maps.device if self._in_maps is not None else self._forward.device
