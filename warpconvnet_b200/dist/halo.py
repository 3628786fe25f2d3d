"""One scene split across ranks by Morton-code range, with a one-voxel halo exchange.

Geometry step (once per scene): all ranks hold the full coordinate list (coordinates are
small: 16 B per voxel), sort it by the 20-bit-per-axis Morton code and own equal-count
contiguous ranges of that order.  A rank searches the 3x3x3 neighbourhood of its owned
voxels in the global set; neighbours it does not own form its halo.  Local input rows are
``[owned ; halo]`` and the neighbour table is re-indexed into that local numbering, so the
convolution kernel only ever reads local memory.  Ranks then tell each other which of their
rows are wanted (index lists, exchanged once).

Per convolution: gather the wanted rows, one ``all_to_all_single`` with per-peer split
sizes, append the received rows after the owned ones, run the ordinary fused convolution.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional

import torch
import torch.distributed as dist
from torch import Tensor


def _default_neighbor_fn(global_coords: Tensor, owned_coords: Tensor) -> Tensor:
    """nbr[27, M_owned] = row of the neighbour in ``global_coords`` or -1 (native kernels)."""
    from ..geometry.coords.search.torch_discrete import generate_kernel_map
    km = generate_kernel_map(global_coords, owned_coords, (1, 1, 1), (3, 3, 3))
    return km.neighbor_table(owned_coords.shape[0])


def _default_morton_fn(xyz: Tensor) -> Tensor:
    from ..geometry.coords.ops.serialization import morton_code
    return morton_code(xyz)


def morton_partition(coords: Tensor, world_size: int, morton_fn: Callable[[Tensor], Tensor] = _default_morton_fn):
    """Sort ``coords [N,4]`` (batch, x, y, z) by Morton code and cut the order into
    ``world_size`` equal-count ranges.  Returns ``(perm, bounds)``: ``coords[perm]`` is the
    global order and rank r owns rows ``bounds[r]:bounds[r+1]`` of it."""
    n = coords.shape[0]
    codes = morton_fn(coords[:, 1:].contiguous())
    perm = torch.argsort(codes, stable=True)
    bounds = [(n * r) // world_size for r in range(world_size + 1)]
    return perm, bounds


@dataclass
class HaloPlan:
    rank: int
    world_size: int
    num_owned: int
    num_halo: int
    nbr_local: Tensor                 # int32 [27, num_owned] indices into [owned ; halo]
    halo_global: Tensor               # int64 [num_halo] rows of the global order, ascending
    recv_counts: List[int]            # halo rows arriving from each peer (ascending peer = ascending row)
    send_counts: List[int]            # rows each peer wants from this rank
    send_index: Tensor                # int64 [sum(send_counts)] owned-local rows, grouped by peer
    interior_rows: Optional[Tensor] = None   # int32: owned rows whose window holds no halo row
    boundary_rows: Optional[Tensor] = None   # int32: the other owned rows
    kernel_map: object = field(default=None, repr=False)
    _split_maps: object = field(default=None, repr=False)
    _comm_stream: object = field(default=None, repr=False)

    @property
    def num_local(self) -> int:
        return self.num_owned + self.num_halo

    def new_local(self, channels: int, dtype: torch.dtype, device) -> Tensor:
        """A ``[owned ; halo]`` feature buffer.  A layer that writes its result into the first
        ``num_owned`` rows of the next layer's buffer never copies the owned rows."""
        return torch.empty((self.num_local, channels), dtype=dtype, device=device)

    def exchange_into(self, local: Tensor, group=None) -> None:
        """Fill the halo rows of ``local`` from the peers' owned rows: gather what they want from
        ``local[:num_owned]``, one all-to-all with per-peer split sizes."""
        if self.world_size <= 1 or (self.num_halo == 0 and len(self.send_index) == 0):
            return
        owned = local[:self.num_owned]
        send = owned[self.send_index] if len(self.send_index) else owned[:0]
        dist.all_to_all_single(local[self.num_owned:], send.contiguous(), self.recv_counts, self.send_counts,
                               group=group)

    def exchange(self, owned_feats: Tensor, group=None) -> Tensor:
        """[owned ; halo] feature rows in a new buffer (copies the owned rows)."""
        local = self.new_local(owned_feats.shape[1], owned_feats.dtype, owned_feats.device)
        local[:self.num_owned] = owned_feats
        self.exchange_into(local, group=group)
        return local

    def split_maps(self):
        """(interior map, boundary map): the local neighbour table restricted to the owned rows that
        need no halo row and to those that do.  Built once per plan."""
        if self._split_maps is None:
            from ..geometry.coords.search.search_results import IntSearchResult
            maps = []
            for rows in (self.interior_rows, self.boundary_rows):
                nbr = self.nbr_local[:, rows.long()].contiguous()
                maps.append(IntSearchResult.from_neighbor_table(nbr, self.num_local, None, None))
            self._split_maps = tuple(maps)
        return self._split_maps


def plan_halo(global_coords_sorted: Tensor, bounds: List[int], rank: int, world_size: int, group=None,
              neighbor_fn: Callable[[Tensor, Tensor], Tensor] = _default_neighbor_fn) -> HaloPlan:
    """Halo and local neighbour table of ``rank`` for a 3x3x3 stride-1 convolution.
    ``global_coords_sorted`` is the Morton-ordered coordinate list every rank holds."""
    lo, hi = bounds[rank], bounds[rank + 1]
    owned = global_coords_sorted[lo:hi].contiguous()
    nbr = neighbor_fn(global_coords_sorted, owned).long()  # global rows, -1 = absent
    foreign = (nbr >= 0) & ((nbr < lo) | (nbr >= hi))
    halo_global = torch.unique(nbr[foreign])  # sorted ascending
    # local numbering: owned rows first (global row - lo), then the halo rows in ascending global order
    local = torch.where(nbr >= 0, nbr - lo, nbr)
    if halo_global.numel():
        pos = torch.searchsorted(halo_global, nbr[foreign])
        local[foreign] = (hi - lo) + pos
    nbr_local = local.to(torch.int32).contiguous()
    # who owns each halo row
    b = torch.tensor(bounds, device=halo_global.device, dtype=torch.long)
    owner = torch.searchsorted(b, halo_global, right=True) - 1
    recv_counts = torch.bincount(owner, minlength=world_size).tolist() if halo_global.numel() else [0] * world_size
    # tell every peer which of its rows are wanted
    if world_size > 1:
        counts_t = torch.tensor(recv_counts, dtype=torch.long, device=halo_global.device)
        send_counts_t = torch.empty_like(counts_t)
        dist.all_to_all_single(send_counts_t, counts_t, group=group)
        send_counts = send_counts_t.tolist()
        wanted = torch.empty(int(sum(send_counts)), dtype=torch.long, device=halo_global.device)
        dist.all_to_all_single(wanted, halo_global.contiguous(), send_counts, recv_counts, group=group)
        send_index = wanted - lo
    else:
        send_counts, send_index = [0], torch.empty(0, dtype=torch.long, device=halo_global.device)
    needs_halo = foreign.any(dim=0)
    rows = torch.arange(hi - lo, device=nbr.device, dtype=torch.int32)
    return HaloPlan(rank, world_size, hi - lo, int(halo_global.numel()), nbr_local, halo_global, recv_counts,
                    send_counts, send_index, interior_rows=rows[~needs_halo].contiguous(),
                    boundary_rows=rows[needs_halo].contiguous())


def partitioned_conv(feats: Tensor, weight: Tensor, plan: HaloPlan, epilogue=None, group=None,
                     overlap: bool = True, out: Optional[Tensor] = None) -> Tensor:
    """3x3x3 stride-1 convolution of the rows this rank owns.

    ``feats`` is either the owned rows ``[num_owned, C]`` (copied into a new ``[owned ; halo]``
    buffer) or such a buffer ``[num_local, C]`` from :meth:`HaloPlan.new_local` whose owned rows are
    filled (nothing is copied; its halo rows are overwritten).  With ``overlap`` the halo exchange
    runs on a stream of its own while the convolution of the interior rows — those whose window
    holds no halo row — is already running; the few boundary rows follow once the halo has
    arrived.  Every output row is computed by the same arithmetic either way, so the result is
    bit-identical to the single-GPU convolution run in one pass (``split_k=1``: the launches here
    never divide the kernel offsets among CTAs, which would regroup the fp32 sums of small launches
    such as the boundary rows).  ``out`` (``[num_owned, C_out]``, may be the owned
    rows of the next layer's buffer) receives the result."""
    from ..geometry.coords.search.search_results import IntSearchResult
    from ..nn.functional.sparse_conv import ConvEpilogue, sparse_conv_fused
    if feats.shape[0] == plan.num_local and plan.num_halo > 0:
        local = feats
    else:
        assert feats.shape[0] == plan.num_owned, "features must be the owned rows or an [owned ; halo] buffer"
        local = plan.new_local(feats.shape[1], feats.dtype, feats.device)
        local[:plan.num_owned] = feats
    ep = epilogue or ConvEpilogue()
    assert ep.out_rows is None and ep.out is None, "use the out= argument"
    c_out = weight.shape[2]
    if out is None:
        out = torch.empty((plan.num_owned, c_out), dtype=local.dtype, device=local.device)
    # (a residual is read at the output row, which a launch over a subset of rows cannot say: one launch then)
    use_overlap = (overlap and plan.world_size > 1 and plan.interior_rows is not None and ep.residual is None
                   and len(plan.boundary_rows) > 0 and len(plan.interior_rows) > 0)
    if not use_overlap:
        plan.exchange_into(local, group=group)
        if plan.kernel_map is None:
            plan.kernel_map = IntSearchResult.from_neighbor_table(plan.nbr_local, plan.num_local, None, None)
        sparse_conv_fused(local, weight, plan.kernel_map, plan.num_owned, split_k=1,
                          epilogue=ConvEpilogue(ep.scale, ep.shift, ep.residual, ep.relu, None, out))
        return out
    if plan._comm_stream is None:
        plan._comm_stream = torch.cuda.Stream(local.device)
    main, side = torch.cuda.current_stream(local.device), plan._comm_stream
    ready, arrived = torch.cuda.Event(), torch.cuda.Event()
    ready.record(main)
    # the exchange is enqueued first so that its (small) kernels get multiprocessors before the
    # persistent convolution kernel occupies all of them
    with torch.cuda.stream(side):
        side.wait_event(ready)
        plan.exchange_into(local, group=group)
        arrived.record(side)
    local.record_stream(side)
    interior, boundary = plan.split_maps()
    for kmap, rows, wait in ((interior, plan.interior_rows, False), (boundary, plan.boundary_rows, True)):
        if wait:
            main.wait_event(arrived)
        sparse_conv_fused(local, weight, kmap, len(rows), split_k=1,
                          epilogue=ConvEpilogue(ep.scale, ep.shift, None, ep.relu, rows, out))
    return out
