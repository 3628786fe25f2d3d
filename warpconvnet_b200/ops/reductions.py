"""Row reductions over a kernel map (warpconvnet/ops/reductions.py:13-70).

The reference reduces a CSR of gathered rows with ``torch_scatter.segment_csr``; here the
reduction runs straight over the dense neighbour table in one native launch
(``wcn_row_reduce``): output row m reduces the input rows ``nbr[k][m] >= 0``.
"""
from __future__ import annotations

from enum import Enum
from typing import Union

import torch
from torch import Tensor

from .._native import check, dtype_code, lib, ptr, require_cuda, stream_ptr
from ..geometry.coords.search.search_results import IntSearchResult


class REDUCTIONS(Enum):
    MIN = "min"
    MAX = "max"
    MEAN = "mean"
    SUM = "sum"
    MUL = "mul"
    VAR = "var"
    STD = "std"
    RANDOM = "random"


_NATIVE_OP = {REDUCTIONS.MIN: 0, REDUCTIONS.MAX: 1, REDUCTIONS.SUM: 2, REDUCTIONS.MEAN: 3, REDUCTIONS.MUL: 4}


def _native_reduce(features: Tensor, nbr: Tensor, op: int) -> Tensor:
    K, M = nbr.shape
    out = torch.empty((M, features.shape[1]), dtype=features.dtype, device=features.device)
    check(lib().wcn_row_reduce(ptr(features), ptr(nbr), M, K, features.shape[1], dtype_code(features.dtype), op,
                               ptr(out), stream_ptr(features.device)), "wcn_row_reduce")
    return out


@torch.no_grad()
def neighbor_reduction(features: Tensor, kernel_map: IntSearchResult, num_out: int,
                       reduction: Union[REDUCTIONS, str], eps: float = 1e-6) -> Tensor:
    """``out[m] = reduction over the neighbours of output row m`` (rows without a neighbour: 0).
    ``var`` / ``std`` follow the reference: mean of squares minus squared mean (+ eps under the root);
    ``random`` picks one neighbour per row uniformly."""
    if isinstance(reduction, str):
        reduction = REDUCTIONS(reduction)
    require_cuda(features, "features")
    if features.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise ValueError(f"unsupported feature dtype {features.dtype}")
    x = features.contiguous()
    nbr = kernel_map.neighbor_table(num_out)
    if reduction in _NATIVE_OP:
        return _native_reduce(x, nbr, _NATIVE_OP[reduction])
    if reduction in (REDUCTIONS.VAR, REDUCTIONS.STD):
        mean = _native_reduce(x, nbr, _NATIVE_OP[REDUCTIONS.MEAN])
        var = _native_reduce(x * x, nbr, _NATIVE_OP[REDUCTIONS.MEAN]) - mean * mean
        return var if reduction == REDUCTIONS.VAR else torch.sqrt(var + eps)
    if reduction == REDUCTIONS.RANDOM:
        present = nbr >= 0
        count = present.sum(0)
        pick = (torch.rand(num_out, device=x.device) * count).floor().long().clamp_(min=0)
        rank = present.long().cumsum(0) - 1                      # rank of each present neighbour in its column
        chosen = (present & (rank == pick.unsqueeze(0))).float().argmax(0)
        idx = nbr.gather(0, chosen.unsqueeze(0)).squeeze(0).long()
        out = x[idx.clamp_(min=0)]
        out[count == 0] = 0
        return out
    raise ValueError(f"Invalid reduction: {reduction}")
