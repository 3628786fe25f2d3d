"""``Sequential`` for mixed geometry / tensor layers (warpconvnet/nn/modules/sequential.py:14-62)
with one addition: in eval mode a run ``SparseConv -> BatchNorm1d [-> ReLU]`` is
executed as ONE kernel (convolution with the folded BatchNorm, an optional
residual and the ReLU in its epilogue).  Training mode and every other layer
pattern run layer by layer exactly like the reference.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
from torch import Tensor

from ...geometry.base.geometry import Geometry
from ..functional.sparse_conv import ConvEpilogue
from .activations import ReLU as GeometryReLU
from .base_module import BaseSpatialModule
from .normalizations import BatchNorm as GeometryBatchNorm
from .sparse_conv import SpatiallySparseConv


def run_forward(module: nn.Module, x, in_sf: Geometry):
    if isinstance(module, BaseSpatialModule) and isinstance(x, Geometry):
        return module(x), in_sf
    if not isinstance(module, BaseSpatialModule) and isinstance(x, Geometry):
        in_sf = x
        x = module(x.feature_tensor)
    elif isinstance(x, Tensor) and isinstance(module, BaseSpatialModule):
        x = module(in_sf.replace(batched_features=x))
    else:
        x = module(x)
    return x, in_sf


def fold_batchnorm(bn: nn.BatchNorm1d):
    """Eval-mode BatchNorm as y = x * scale + shift (fp32 vectors), cached on the
    module until one of its tensors changes."""
    tensors = (bn.running_var, bn.running_mean, bn.weight, bn.bias)
    tag = tuple((t.data_ptr(), t._version) if t is not None else None for t in tensors)
    hit = bn.__dict__.get("_wcn_folded")
    if hit is not None and hit[0] == tag:
        return hit[1], hit[2]
    scale, shift = _fold_batchnorm(bn)
    bn.__dict__["_wcn_folded"] = (tag, scale, shift)
    return scale, shift


def _fold_batchnorm(bn: nn.BatchNorm1d):
    var = bn.running_var.detach().float()
    mean = bn.running_mean.detach().float()
    gamma = bn.weight.detach().float() if bn.weight is not None else torch.ones_like(var)
    beta = bn.bias.detach().float() if bn.bias is not None else torch.zeros_like(var)
    scale = gamma * torch.rsqrt(var + bn.eps)
    return scale, beta - mean * scale


def _as_bn(m) -> Optional[nn.BatchNorm1d]:
    if isinstance(m, nn.BatchNorm1d):
        return m
    if isinstance(m, GeometryBatchNorm):
        return m.norm
    return None


def _is_relu(m) -> bool:
    return isinstance(m, (nn.ReLU, GeometryReLU))


class Sequential(nn.Sequential, BaseSpatialModule):
    def forward(self, x: Geometry, residual: Optional[Tensor] = None, final_relu: bool = False,
                out: Optional[Tensor] = None):
        """``residual`` / ``final_relu`` (additions to the reference signature) are
        applied after the last layer: ``relu(out + residual)``; when the tail of the
        sequence is a fusable conv-BN run they ride in its epilogue.  ``out`` (inference
        only) is a preallocated ``[M, C]`` destination for the features of the result, e.g.
        a column block of a concatenation buffer; it needs that fused tail."""
        assert isinstance(x, Geometry), f"Expected Geometry, got {type(x)}"
        mods = list(self)
        in_sf = x
        i = 0
        fused_tail = False
        can_fuse = not torch.is_grad_enabled() or not any(p.requires_grad for p in self.parameters())
        while i < len(mods):
            m = mods[i]
            bn = _as_bn(mods[i + 1]) if i + 1 < len(mods) else None
            if (can_fuse and isinstance(m, SpatiallySparseConv) and isinstance(x, Geometry) and bn is not None
                    and not bn.training and bn.track_running_stats and not m.generative):
                j = i + 2
                relu = j < len(mods) and _is_relu(mods[j])
                if relu:
                    j += 1
                elif j < len(mods) and isinstance(mods[j], nn.Identity):
                    j += 1
                scale, shift = fold_batchnorm(bn)
                ep = ConvEpilogue(scale=scale, shift=shift, relu=relu)
                if j == len(mods) and (residual is not None or final_relu) and not relu:
                    ep.residual, ep.relu = residual, final_relu
                    fused_tail = True
                if j == len(mods) and out is not None and (fused_tail or (residual is None and not final_relu)):
                    ep.out, out = out, None
                x = m(x, epilogue=ep)
                i = j
                continue
            x, in_sf = run_forward(m, x, in_sf)
            i += 1
        if isinstance(x, Tensor):
            x = in_sf.replace(batched_features=x)
        if not fused_tail and (residual is not None or final_relu):
            f = x.feature_tensor
            if residual is not None:
                f = f + residual
            if final_relu:
                f = torch.relu(f)
            x = x.replace(batched_features=f)
        if out is not None:  # no fused tail took it: copy
            out.copy_(x.feature_tensor)
            x = x.replace(batched_features=out)
        return x
