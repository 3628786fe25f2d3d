"""Batch index / offsets helpers (warpconvnet/geometry/coords/ops/batch_index.py:23-36,111-161)."""
import torch
from torch import Tensor


@torch.no_grad()
def batch_index_from_offset(offsets: Tensor) -> Tensor:
    """[0,0,..,1,1,..] for offsets [0, n0, n0+n1, ...]."""
    assert len(offsets) > 1, "offsets must have at least two elements. [0, N] for batch size 1"
    counts = torch.diff(offsets)
    return torch.arange(len(counts), device=offsets.device, dtype=torch.long).repeat_interleave(counts)


@torch.no_grad()
def batch_index_on(offsets: Tensor, n: int, device, dtype=torch.int32) -> Tensor:
    """Batch index of rows 0..n-1 on ``device``: one bucketize of an arange against the
    batch boundaries (no host synchronisation, no repeat_interleave)."""
    from ...._native import small_to_device
    bounds = (small_to_device(offsets[1:], device, torch.int64) if torch.device(device).type == "cuda"
              else offsets[1:].to(device=device, dtype=torch.int64))
    return torch.bucketize(torch.arange(n, device=device, dtype=torch.int64), bounds, right=True).to(dtype)


@torch.no_grad()
def batch_indexed_coordinates(batched_coords: Tensor, offsets: Tensor) -> Tensor:
    """Prepend the batch index column: [N, D] -> [N, D+1]."""
    batch_index = batch_index_on(offsets, batched_coords.shape[0], batched_coords.device, batched_coords.dtype)
    return torch.cat([batch_index.unsqueeze(1), batched_coords], dim=1)


@torch.no_grad()
def offsets_from_batch_index(batch_index: Tensor) -> Tensor:
    """CPU offsets [B+1] from a (batch-sorted) batch index column."""
    counts = torch.bincount(batch_index).cpu()
    return torch.cat([torch.zeros(1, dtype=torch.int32), counts.cumsum(dim=0)], dim=0)
