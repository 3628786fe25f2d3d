"""Scene-group sharding of a batch: rank r takes a contiguous run of scenes."""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch

from ..geometry.coords.integer import IntCoords
from ..geometry.features.cat import CatFeatures
from ..geometry.types.voxels import Voxels


def split_scene_groups(offsets: Sequence[int], world_size: int) -> List[Tuple[int, int]]:
    """Cut ``B`` scenes (``offsets`` has B+1 entries) into ``world_size`` contiguous groups
    ``[(first_scene, last_scene_exclusive), ...]`` with voxel counts as even as contiguity
    allows: group g ends at the scene boundary nearest to g+1 shares of the total, and no
    group is empty while there are at least as many scenes as ranks.
    Every scene belongs to exactly one group; groups may be empty when B < world_size."""
    offs = [int(o) for o in offsets]
    b = len(offs) - 1
    assert b >= 0 and world_size >= 1
    total = offs[-1] - offs[0]
    cuts = [0]
    for g in range(1, world_size):
        target = offs[0] + total * g / world_size
        lo, hi = cuts[-1], b
        if b >= world_size:  # leave at least one scene for this group and for each later one
            lo, hi = cuts[-1] + 1, b - (world_size - g)
        best = min(range(lo, hi + 1), key=lambda i: (abs(offs[i] - target), i))
        cuts.append(best)
    cuts.append(b)
    return [(cuts[g], cuts[g + 1]) for g in range(world_size)]


def shard_voxels(voxels: Voxels, rank: int, world_size: int) -> Voxels:
    """The scenes of ``voxels`` that belong to ``rank`` (batch indices renumbered from 0).
    The kernel-map cache is not carried over: maps index rows of the full batch."""
    first, last = split_scene_groups(voxels.offsets.tolist(), world_size)[rank]
    offs = voxels.offsets.long()
    lo, hi = int(offs[first]), int(offs[last])
    new_offsets = (offs[first:last + 1] - offs[first]).clone()
    extras = voxels.extra_attributes
    extras.pop("_cache", None)
    for stale in ("code", "perm"):
        extras.pop(stale, None)
    return Voxels(IntCoords(voxels.coordinate_tensor[lo:hi], new_offsets, tensor_stride=voxels.tensor_stride),
                  CatFeatures(voxels.feature_tensor[lo:hi], new_offsets), **extras)
