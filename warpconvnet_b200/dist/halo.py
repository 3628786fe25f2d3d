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
    kernel_map: object = field(default=None, repr=False)

    @property
    def num_local(self) -> int:
        return self.num_owned + self.num_halo

    def exchange(self, owned_feats: Tensor, group=None) -> Tensor:
        """[owned ; halo] feature rows: gather what the peers want, one all-to-all."""
        c = owned_feats.shape[1]
        local = torch.empty((self.num_local, c), dtype=owned_feats.dtype, device=owned_feats.device)
        local[:self.num_owned] = owned_feats
        send = owned_feats[self.send_index] if len(self.send_index) else owned_feats[:0]
        recv = local[self.num_owned:]
        if self.world_size > 1:
            dist.all_to_all_single(recv, send.contiguous(), self.recv_counts, self.send_counts, group=group)
        return local


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
    return HaloPlan(rank, world_size, hi - lo, int(halo_global.numel()), nbr_local, halo_global, recv_counts,
                    send_counts, send_index)


def partitioned_conv(owned_feats: Tensor, weight: Tensor, plan: HaloPlan, epilogue=None, group=None) -> Tensor:
    """3x3x3 stride-1 convolution of the rows this rank owns: halo exchange + fused kernel."""
    from ..geometry.coords.search.search_results import IntSearchResult
    from ..nn.functional.sparse_conv import sparse_conv_fused
    if plan.kernel_map is None:
        plan.kernel_map = IntSearchResult.from_neighbor_table(plan.nbr_local, plan.num_local, None, None)
    local = plan.exchange(owned_feats, group=group)
    return sparse_conv_fused(local, weight, plan.kernel_map, plan.num_owned, epilogue=epilogue)
