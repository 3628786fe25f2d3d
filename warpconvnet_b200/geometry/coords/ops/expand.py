"""Coordinates reached by a kernel window from a coordinate set, the output support of a
generative convolution (warpconvnet/geometry/coords/ops/expand.py:17-64).

The reference grows the set offset batch by offset batch, rebuilding its hash table each time;
here all ``N * K`` candidates are formed at once and made distinct by one pass of the native
unique kernels.  The rows come out batch-sorted, the input rows first inside each batch item
(only the SET is defined by the reference: its order depends on hash-table slots).
"""
from __future__ import annotations

from typing import Tuple

import torch
from torch import Tensor

from ..search.torch_discrete import kernel_offsets_from_size
from .batch_index import offsets_from_batch_index
from .stride import unique_strided_rows


@torch.no_grad()
def expand_coords(batch_indexed_coords: Tensor, kernel_size: Tuple[int, ...],
                  kernel_dilation: Tuple[int, ...]) -> Tuple[Tensor, Tensor]:
    """``unique(coords + offset_k for every k)``, which contains ``coords`` itself for odd windows.
    Returns ``(rows [M, 4] int32, CPU offsets [B + 1])``."""
    c = batch_indexed_coords.to(torch.int32)
    offsets = kernel_offsets_from_size(kernel_size, kernel_dilation, device=c.device).to(torch.int32)
    centre = (offsets == 0).all(dim=1)
    # the unshifted rows first, so that first-occurrence order starts with the input rows
    order = torch.cat([torch.nonzero(centre).flatten(), torch.nonzero(~centre).flatten()])
    cand = (c.unsqueeze(0) + offsets[order].unsqueeze(1)).reshape(-1, c.shape[1]).contiguous()
    if not bool(centre.any()):
        cand = torch.cat([c, cand], dim=0)
    rows, _, _ = unique_strided_rows(cand)
    rows = rows[torch.argsort(rows[:, 0], stable=True)]
    return rows.contiguous(), offsets_from_batch_index(rows[:, 0])
