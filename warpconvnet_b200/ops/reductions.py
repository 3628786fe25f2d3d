"""Row reductions over a kernel map (warpconvnet/ops/reductions.py:13-70).

The reference reduces a CSR of gathered rows with ``torch_scatter.segment_csr``; here the
reduction runs straight over the dense neighbour table in one native launch
(``wcn_row_reduce``): output row m reduces the input rows ``nbr[k][m] >= 0``.  The reductions
are differentiable like the reference's (its ``segment_csr`` is an autograd op): sum and mean
send the output gradient back through the transposed table with the same kernel, max and min
send it to the row that attained the extremum.
"""
from __future__ import annotations

from enum import Enum
from typing import Union

import torch
from torch import Tensor

from .._native import check, device_status, dtype_code, lib, ptr, require_cuda, stream_ptr
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
    dev = features.device
    out = torch.empty((M, features.shape[1]), dtype=features.dtype, device=dev)
    check(lib().wcn_row_reduce(ptr(features), features.shape[0], ptr(nbr), M, K, features.shape[1],
                               dtype_code(features.dtype), op, ptr(out), ptr(device_status(dev)), stream_ptr(dev)),
          "wcn_row_reduce")
    return out


class _RowReduce(torch.autograd.Function):
    """``wcn_row_reduce`` with a backward pass.

    sum / mean: ``dX[i] = sum over (k, m) with nbr[k][m] == i of dY[m] (/ count[m])`` — the same
    kernel over the transposed table.  max / min: the gradient of output row m goes, per channel,
    to the first neighbour (ascending offset) whose value equals the result, as ``segment_csr``'s
    arg-extremum does.  mul has no backward here."""

    @staticmethod
    def forward(ctx, features: Tensor, kernel_map: IntSearchResult, num_out: int, op: int) -> Tensor:
        x = features.contiguous()
        out = _native_reduce(x, kernel_map.neighbor_table(num_out), op)
        ctx.kernel_map, ctx.num_out, ctx.op = kernel_map, num_out, op
        ctx.save_for_backward(x, out)
        return out

    @staticmethod
    def backward(ctx, grad_out: Tensor):
        x, out = ctx.saved_tensors
        km, M, op = ctx.kernel_map, ctx.num_out, ctx.op
        g = grad_out.contiguous()
        nbr = km.neighbor_table(M)
        if op in (_NATIVE_OP[REDUCTIONS.SUM], _NATIVE_OP[REDUCTIONS.MEAN]):
            if op == _NATIVE_OP[REDUCTIONS.MEAN]:
                count = (nbr >= 0).sum(0).clamp_(min=1).to(g.dtype)
                g = (g / count.unsqueeze(1)).contiguous()
            nbr_t = km.swapped(num_in=x.shape[0]).neighbor_table(x.shape[0])
            return _native_reduce(g, nbr_t, _NATIVE_OP[REDUCTIONS.SUM]), None, None, None
        if op in (_NATIVE_OP[REDUCTIONS.MAX], _NATIVE_OP[REDUCTIONS.MIN]):
            gx = torch.zeros_like(x)
            taken = torch.zeros_like(out, dtype=torch.bool)
            for k in range(nbr.shape[0]):
                rows = nbr[k].long()
                have = rows >= 0
                src = rows.clamp(min=0)
                hit = have.unsqueeze(1) & (x[src] == out) & ~taken
                gx.index_add_(0, src, torch.where(hit, g, torch.zeros_like(g)))
                taken |= hit
            return gx, None, None, None
        raise NotImplementedError("the 'mul' reduction has no backward pass")


def neighbor_reduction(features: Tensor, kernel_map: IntSearchResult, num_out: int,
                       reduction: Union[REDUCTIONS, str], eps: float = 1e-6) -> Tensor:
    """``out[m] = reduction over the neighbours of output row m`` (rows without a neighbour: 0).
    ``var`` / ``std`` follow the reference: mean of squares minus squared mean (+ eps under the root);
    ``random`` picks one neighbour per row uniformly.  Differentiable with respect to ``features``."""
    if isinstance(reduction, str):
        reduction = REDUCTIONS(reduction)
    require_cuda(features, "features")
    if features.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise ValueError(f"unsupported feature dtype {features.dtype}")
    tracked = torch.is_grad_enabled() and features.requires_grad

    def native(x: Tensor, red: REDUCTIONS) -> Tensor:
        if tracked:
            return _RowReduce.apply(x, kernel_map, num_out, _NATIVE_OP[red])
        return _native_reduce(x.contiguous(), kernel_map.neighbor_table(num_out), _NATIVE_OP[red])

    if reduction in _NATIVE_OP:
        return native(features, reduction)
    if reduction in (REDUCTIONS.VAR, REDUCTIONS.STD):
        mean = native(features, REDUCTIONS.MEAN)
        var = native(features * features, REDUCTIONS.MEAN) - mean * mean
        return var if reduction == REDUCTIONS.VAR else torch.sqrt(var + eps)
    if reduction == REDUCTIONS.RANDOM:
        with torch.no_grad():
            nbr = kernel_map.neighbor_table(num_out)
            present = nbr >= 0
            count = present.sum(0)
            pick = (torch.rand(num_out, device=features.device) * count).floor().long().clamp_(min=0)
            rank = present.long().cumsum(0) - 1                      # rank of each present neighbour in its column
            chosen = (present & (rank == pick.unsqueeze(0))).float().argmax(0)
            idx = nbr.gather(0, chosen.unsqueeze(0)).squeeze(0).long().clamp_(min=0)
        out = features[idx]                                          # differentiable gather
        return out * (count > 0).to(out.dtype).unsqueeze(1)
    raise ValueError(f"Invalid reduction: {reduction}")
