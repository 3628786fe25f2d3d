"""Multi-GPU use of the sparse-convolution path: one process per GPU.

``sharding``  batches of scenes split into contiguous scene groups, one per rank, no
              communication (every key carries its batch index, so scenes never interact).
``halo``      one huge scene split by Morton-code range; before a 3x3x3 convolution each rank
              receives the feature rows of the one-voxel halo of its range with one
              ``all_to_all_single`` (NCCL over NVLink on GPUs, gloo in the CPU tests).
The reference has no counterpart: it contains no collective (its only distributed code is a
user-side FSDP wrapper in ``tests/test_fsdp.py``).
"""
from .halo import HaloPlan, morton_partition, partitioned_conv, plan_halo
from .sharding import shard_voxels, split_scene_groups
