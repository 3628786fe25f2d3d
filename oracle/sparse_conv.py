"""torch-CPU restatement of the reference's explicit-GEMM sparse convolution,
the BatchNorm / ReLU / residual chain and the MinkUNet forward built on them.

TEST INFRASTRUCTURE ONLY (checker and timed CPU baseline); the product package
never imports this file.  Kernel maps come from ``oracle/kernel_map.py``.

Parity: pinned — :func:`explicit_gemm_forward` is compared with the reference's
``_explicit_gemm_forward_logic`` run on the same CPU tensors when the golden
fixtures are generated (``tests/golden/make_golden.py``) and the fixtures are
replayed in ``tests/test_oracle_pins.py``.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import numpy as np
import torch

from . import kernel_map as km


def explicit_gemm_forward(feats: torch.Tensor, weight: torch.Tensor, in_maps, out_maps, offsets,
                          identity_index: Optional[int], num_out: int,
                          compute_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``out = X @ W[c]`` for the identity offset (else zeros), then for every
    other offset ``out[out_map_k] += X[in_map_k] @ W[k]``; result cast back to
    the input dtype.  Restates ``_explicit_gemm_forward_logic``
    (warpconvnet/nn/functional/sparse_conv.py:281-311)."""
    x = feats if compute_dtype is None else feats.to(compute_dtype)
    w = weight if compute_dtype is None else weight.to(compute_dtype)
    in_maps = torch.as_tensor(np.asarray(in_maps), dtype=torch.long)
    out_maps = torch.as_tensor(np.asarray(out_maps), dtype=torch.long)
    offsets = np.asarray(offsets)
    if identity_index is not None:
        out = x @ w[identity_index]
    else:
        out = torch.zeros(num_out, w.shape[-1], dtype=x.dtype)
    for k in range(len(offsets) - 1):
        if k == identity_index:
            continue
        s, e = int(offsets[k]), int(offsets[k + 1])
        if e == s:
            continue
        out[out_maps[s:e]] += x[in_maps[s:e]] @ w[k]
    return out.to(feats.dtype)


def batchnorm_eval(x: torch.Tensor, weight, bias, running_mean, running_var, eps: float = 1e-5):
    """``nn.BatchNorm1d`` in eval mode (the reference's BatchNorm wrapper,
    warpconvnet/nn/modules/normalizations.py:49-63, applies it to the feature
    tensor): per-channel affine from the running statistics."""
    return torch.nn.functional.batch_norm(x, running_mean, running_var, weight, bias, False, 0.0, eps)


# --------------------------------------------------------------------------- network


class _Geom:
    """Coordinates [N,4] (NumPy) + features (torch) + a per-network map cache
    keyed like the reference's IntSearchCacheKey (kernel, transposed, in/out
    per-batch counts; warpconvnet/geometry/coords/search/cache.py:84-142)."""

    def __init__(self, coords, feats, cache):
        self.coords, self.feats, self.cache = coords, feats, cache

    def counts(self):
        return tuple(np.bincount(self.coords[:, 0]).tolist())


def _conv(g: _Geom, weight: torch.Tensor, kernel: int, stride: int = 1, transposed: bool = False,
          out_geom: Optional[_Geom] = None) -> _Geom:
    """``spatially_sparse_conv`` (warpconvnet/nn/functional/sparse_conv.py:1662-1805),
    explicit-GEMM algorithm, STRIDE_ONLY mode."""
    if kernel == 1 and stride == 1:
        return _Geom(g.coords, g.feats @ weight[0], g.cache)  # :1714-1721
    ks, st = (kernel,) * 3, (stride,) * 3
    if transposed:
        out_coords = out_geom.coords
        key = ("T", ks, g.counts(), out_geom.counts())
        if key not in g.cache:
            fkey = ("F", ks, out_geom.counts(), g.counts())
            if fkey in g.cache:  # :1916-1939: forward map with in/out swapped
                fi, fo, fofs, _ = g.cache[fkey]
                g.cache[key] = (fo, fi, fofs, None)
            else:
                g.cache[key] = km.transposed_kernel_map(g.coords, out_coords, st, ks)
    else:
        out_coords = g.coords if stride == 1 else km.stride_coords(g.coords, st)[0]
        key = ("F", ks, g.counts(), tuple(np.bincount(out_coords[:, 0]).tolist()))
        if key not in g.cache:
            g.cache[key] = km.generate_kernel_map(g.coords, out_coords, st, ks)
    im, om, ofs, iden = g.cache[key]
    out = explicit_gemm_forward(g.feats, weight, im, om, ofs, iden, len(out_coords))
    return _Geom(out_coords, out, g.cache)


def _bn(sd, prefix, x):
    return batchnorm_eval(x, sd[prefix + ".weight"], sd[prefix + ".bias"], sd[prefix + ".running_mean"],
                          sd[prefix + ".running_var"])


def _conv_block(sd, prefix, g, kernel, stride=1, act=True):
    # ConvBlock = SparseConv3d(bias=False) -> BatchNorm1d -> ReLU|Identity (examples/mink_unet.py:25-47)
    g = _conv(g, sd[prefix + ".0.weight"], kernel, stride)
    x = _bn(sd, prefix + ".1", g.feats)
    return _Geom(g.coords, torch.relu(x) if act else x, g.cache)


def _basic_block(sd, prefix, g):
    # BasicBlock (examples/mink_unet.py:86-141)
    out = _conv_block(sd, prefix + ".conv1", g, 3)
    out = _conv_block(sd, prefix + ".conv2", out, 3, act=False)
    identity = g
    if (prefix + ".downsample.0.weight") in sd:
        identity = _conv_block(sd, prefix + ".downsample", g, 1, act=False)
    return _Geom(out.coords, torch.relu(out.feats + identity.feats), g.cache)


def _conv_tr_block(sd, prefix, g, skip):
    # ConvTrBlock (examples/mink_unet.py:50-83)
    out = _conv(g, sd[prefix + ".conv_tr.weight"], 2, 2, transposed=True, out_geom=skip)
    return _Geom(out.coords, torch.relu(_bn(sd, prefix + ".norm_act.0", out.feats)), g.cache)


def basic_block(state_dict: Dict[str, torch.Tensor], prefix: str, coords: np.ndarray, feats: torch.Tensor) -> torch.Tensor:
    """One residual block of the network (examples/mink_unet.py:86-141) on its own: the features it
    produces for the rows of ``coords``.  ``prefix`` names the block in the state dict
    ("block3.1"); parameters are used in the dtype of ``feats``."""
    sd = {k: (v.detach().to("cpu").to(feats.dtype) if v.is_floating_point() else v.detach().to("cpu"))
          for k, v in state_dict.items() if k.startswith(prefix + ".")}
    return _basic_block(sd, prefix, _Geom(np.ascontiguousarray(coords, dtype=np.int32), feats, {})).feats


def minkunet_forward(state_dict: Dict[str, torch.Tensor], coords: np.ndarray, feats: torch.Tensor,
                     layers: Sequence[int] = (2, 3, 4, 6, 2, 2, 2, 2), trace: Optional[dict] = None) -> torch.Tensor:
    """MinkUNet forward (examples/mink_unet.py:324-361) on CPU tensors from a
    ``state_dict`` whose parameter names follow the reference model.  ``trace`` (a dict) receives,
    per residual block name, ``(coords, input features, output features)``."""
    sd = {k: v.detach().to("cpu") for k, v in state_dict.items()}
    dtype = feats.dtype
    sd = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in sd.items()}
    g = _Geom(np.ascontiguousarray(coords, dtype=np.int32), feats, {})

    def blocks(name, g, n):
        for i in range(n):
            out = _basic_block(sd, f"{name}.{i}", g)
            if trace is not None:
                trace[f"{name}.{i}"] = (g.coords, g.feats, out.feats)
            g = out
        return g

    out_p1 = _conv_block(sd, "conv0", g, 1)
    out = _conv_block(sd, "conv1", out_p1, 2, 2)
    out_b1p2 = blocks("block1", out, layers[0])
    out = _conv_block(sd, "conv2", out_b1p2, 2, 2)
    out_b2p4 = blocks("block2", out, layers[1])
    out = _conv_block(sd, "conv3", out_b2p4, 2, 2)
    out_b3p8 = blocks("block3", out, layers[2])
    out = _conv_block(sd, "conv4", out_b3p8, 2, 2)
    out = blocks("block4", out, layers[3])

    def up(name, block, out, skip, n):
        out = _conv_tr_block(sd, name, out, skip)
        out = _Geom(out.coords, torch.cat([out.feats, skip.feats], dim=-1), out.cache)
        return blocks(block, out, n)

    out = up("convtr4", "block5", out, out_b3p8, layers[4])
    out = up("convtr5", "block6", out, out_b2p4, layers[5])
    out = up("convtr6", "block7", out, out_b1p2, layers[6])
    out = up("convtr7", "block8", out, out_p1, layers[7])
    return out.feats @ sd["final.weight"][0] + sd["final.bias"]


def window_reduce(feats: np.ndarray, in_maps: np.ndarray, out_maps: np.ndarray, num_out: int,
                  reduction: str) -> np.ndarray:
    """Restates ``sparse_reduce`` (warpconvnet/nn/functional/sparse_pool.py:87-107): the rows
    ``feats[in_maps]`` grouped by ``out_maps`` and reduced per group as ``row_reduction`` /
    ``segment_csr`` do (warpconvnet/ops/reductions.py:36-70); output rows without any input are 0."""
    feats = np.asarray(feats, dtype=np.float64)
    out = np.zeros((num_out, feats.shape[1]), dtype=np.float64)
    order = np.argsort(out_maps, kind="stable")
    o, i = np.asarray(out_maps)[order], np.asarray(in_maps)[order]
    bounds = np.flatnonzero(np.diff(o)) + 1
    starts = np.concatenate([[0], bounds]) if len(o) else np.zeros(0, dtype=np.int64)
    ends = np.concatenate([bounds, [len(o)]]) if len(o) else np.zeros(0, dtype=np.int64)
    for s, e in zip(starts, ends):
        rows = feats[i[s:e]]
        if reduction == "max":
            r = rows.max(0)
        elif reduction == "min":
            r = rows.min(0)
        elif reduction == "sum":
            r = rows.sum(0)
        elif reduction == "mean":
            r = rows.mean(0)
        elif reduction == "mul":
            r = rows.prod(0)
        elif reduction == "var":
            r = (rows ** 2).mean(0) - rows.mean(0) ** 2
        elif reduction == "std":
            r = np.sqrt((rows ** 2).mean(0) - rows.mean(0) ** 2 + 1e-6)
        else:
            raise ValueError(reduction)
        out[o[s]] = r
    return out
