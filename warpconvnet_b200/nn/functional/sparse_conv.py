"""Functional sparse convolution (warpconvnet/nn/functional/sparse_conv.py).

``spatially_sparse_conv`` keeps the reference's signature and semantics
(:1662-1805): the 1x1x1 shortcut, tensor-stride bookkeeping, output-coordinate
selection, the shared kernel-map cache with transposed maps taken from the
forward map (:1808-1996), the explicit / implicit algorithm switch and the bias
add.  Behind it:

* ``explicit_gemm``: per kernel offset, a row-gather kernel, a dense cuBLAS GEMM
  and an owner scatter-add kernel (the reference's algorithm, :281-311);
* ``implicit_gemm`` / ``cutlass_implicit_gemm`` / ``auto``: ONE output-stationary
  kernel over the dense neighbour table — tcgen05 tensor cores for fp16/bf16
  with channel counts it supports, an FP32-pipe kernel otherwise — with bias,
  folded BatchNorm, residual add and ReLU fused into its epilogue when the
  caller passes a :class:`ConvEpilogue`.

There is no auto-tuner and no CPU path.
"""
from __future__ import annotations

import ctypes
import enum
from dataclasses import dataclass
from typing import List, Optional, Tuple, Union

import numpy as np
import torch
from torch import Tensor

from ..._native import (CONV_AUTO, CONV_SIMT, CONV_TCGEN05, LAUNCH_COUNTS, check, device_status, dtype_code, lib, ptr,
                        query_bytes, require_cuda, stream_ptr)
from ...geometry.coords.integer import IntCoords
from ...geometry.coords.ops.serialization import POINT_ORDERING, encode
from ...geometry.coords.ops.expand import expand_coords
from ...geometry.coords.ops.stride import stride_coords
from ...geometry.coords.search.cache import IntSearchCache, IntSearchCacheKey
from ...geometry.coords.search.search_results import IntSearchResult
from ...geometry.coords.search.torch_discrete import generate_kernel_map
from ...geometry.types.voxels import Voxels
from ...utils.ntuple import ntuple
from ...utils.type_cast import _maybe_cast, _min_dtype


class STRIDED_CONV_MODE(enum.Enum):
    REDUCE_AND_STRIDE = "reduce_and_stride"
    STRIDE_ONLY = "stride_only"


class SPARSE_CONV_FWD_ALGO_MODE(enum.Enum):
    EXPLICIT_GEMM = "explicit_gemm"
    IMPLICIT_GEMM = "implicit_gemm"
    CUTLASS_IMPLICIT_GEMM = "cutlass_implicit_gemm"
    AUTO = "auto"


class SPARSE_CONV_BWD_ALGO_MODE(enum.Enum):
    EXPLICIT_GEMM = "explicit_gemm"
    IMPLICIT_GEMM = "implicit_gemm"
    CUTLASS_IMPLICIT_GEMM = "cutlass_implicit_gemm"
    AUTO = "auto"


@dataclass
class ConvEpilogue:
    """Element-wise tail fused into the convolution kernel:
    ``y = conv * scale + shift; y += residual; y = relu(y)`` (each part optional).
    ``scale``/``shift`` are fp32 ``[C_out]`` (an eval-mode BatchNorm folds to
    exactly this; a bias is a shift); ``residual`` is ``[M, C_out]`` in the
    output dtype.  ``out_rows`` (a permutation of ``0..M-1``) stores result row
    ``s`` at row ``out_rows[s]`` of the output, e.g. the ``perm`` of a sorted
    ``Voxels`` to get the rows back in the order they had before the sort; it
    cannot be combined with ``residual``.  With ``out`` given, ``out_rows`` may
    also be distinct rows of a taller ``out`` (a launch over a subset of its rows).  ``out`` is an optional preallocated
    ``[M, C_out]`` destination whose rows may be further apart than ``C_out``
    elements (``out.stride(1) == 1``), e.g. a column block of the buffer a later
    layer reads as the concatenation of two tensors: the convolution then writes
    its half in place and no ``cat`` copy is needed."""

    scale: Optional[Tensor] = None
    shift: Optional[Tensor] = None
    residual: Optional[Tensor] = None
    relu: bool = False
    out_rows: Optional[Tensor] = None
    out: Optional[Tensor] = None


def _normalize_fwd_algo(algo) -> SPARSE_CONV_FWD_ALGO_MODE:
    """Enum | str | list of either -> one algorithm.  A list means "pick the
    best of these" in the reference (:1338-1363); without a tuner the first
    native-kernel entry wins, else the first entry."""
    if isinstance(algo, (list, tuple)):
        items = [_normalize_fwd_algo(a) for a in algo]
        if not items:
            raise ValueError("empty algorithm list")
        for a in items:
            if a != SPARSE_CONV_FWD_ALGO_MODE.EXPLICIT_GEMM:
                return a
        return items[0]
    if isinstance(algo, SPARSE_CONV_FWD_ALGO_MODE):
        return algo
    if isinstance(algo, str):
        try:
            return SPARSE_CONV_FWD_ALGO_MODE(algo.lower())
        except ValueError:
            raise ValueError(f"Unsupported forward algorithm: {algo}")
    if isinstance(algo, enum.Enum) and isinstance(algo.value, str):
        return _normalize_fwd_algo(algo.value)
    raise ValueError(f"Unsupported forward algorithm: {algo}")


# --------------------------------------------------------------------------- kernels


def _gather_rows(src: Tensor, idx: Tensor) -> Tensor:
    dst = torch.empty((idx.shape[0], src.shape[1]), dtype=src.dtype, device=src.device)
    check(lib().wcn_gather_rows(ptr(src), src.shape[0], ptr(idx), ptr(dst), idx.shape[0], src.shape[1],
                                dtype_code(src.dtype), ptr(device_status(src.device)), stream_ptr(src.device)),
          "wcn_gather_rows")
    return dst


def _scatter_add_rows(src: Tensor, idx: Tensor, dst: Tensor) -> None:
    check(lib().wcn_scatter_add_rows(ptr(src), ptr(idx), ptr(dst), dst.shape[0], idx.shape[0], src.shape[1],
                                     dtype_code(src.dtype), ptr(device_status(src.device)), stream_ptr(src.device)),
          "wcn_scatter_add_rows")


def _explicit_gemm_forward_logic(in_features: Tensor, weight: Tensor, kernel_map: IntSearchResult,
                                 num_out_coords: int, compute_dtype: Optional[torch.dtype] = None) -> Tensor:
    """gather -> GEMM -> scatter-add per kernel offset; the identity offset is one
    dense GEMM (reference :281-311)."""
    require_cuda(in_features, "in_features")
    x = _maybe_cast(in_features, compute_dtype).contiguous()
    w = _maybe_cast(weight, compute_dtype).contiguous()
    iden = kernel_map.identity_map_index
    if iden is not None:
        out = torch.matmul(x, w[iden])
    else:
        out = torch.zeros(num_out_coords, w.shape[-1], device=x.device, dtype=x.dtype)
    offsets = kernel_map.offsets
    in_maps, out_maps = kernel_map.in_maps, kernel_map.out_maps
    for k in range(len(kernel_map)):
        if k == iden:
            continue
        s, e = int(offsets[k]), int(offsets[k + 1])
        if e == s:
            continue
        cur = torch.matmul(_gather_rows(x, in_maps[s:e]), w[k])
        _scatter_add_rows(cur, out_maps[s:e], out)
    return out.to(dtype=in_features.dtype)


def _prepared_weight(weight: Tensor, dtype: torch.dtype, algo: int = CONV_AUTO):
    """(weight in ``dtype``, its re-tiled copy for the tensor-core kernel or None).

    Both are cached ON the weight tensor object, tagged with its version counter,
    so an inference loop casts and re-tiles a parameter once and a parameter
    update invalidates the copy."""
    store = weight.__dict__.setdefault("_wcn_prepared", {})
    hit = store.get((dtype, algo))
    if hit is not None and hit[0] == weight._version and hit[1].device == weight.device:
        return hit[1], hit[2]
    w = weight.detach().to(dtype=dtype).contiguous()
    K, c_in, c_out = w.shape
    packed = None
    if algo != CONV_SIMT and w.is_cuda:
        nbytes = query_bytes("wcn_conv_packed_weight_bytes", algo, K, c_in, c_out, dtype_code(dtype))
        if nbytes > 0:
            packed = torch.empty(nbytes, dtype=torch.uint8, device=w.device)
            check(lib().wcn_conv_pack_weight(algo, ptr(w), K, c_in, c_out, dtype_code(dtype), ptr(packed),
                                             stream_ptr(w.device)), "wcn_conv_pack_weight")
    store[(dtype, algo)] = (weight._version, w, packed)
    return w, packed


def _as_f32_on(t: Optional[Tensor], dev: torch.device) -> Optional[Tensor]:
    if t is None:
        return None
    if t.dtype != torch.float32 or t.device != dev:
        t = t.to(device=dev, dtype=torch.float32)
    return t if t.is_contiguous() else t.contiguous()


# Kernel maps with at least this many output rows and this many offsets (at most 32) are run in tile
# order; for 2x2x2 maps building the order costs about what it saves.
TILE_ORDER_MIN_ROWS = 1024
TILE_ORDER_MIN_OFFSETS = 9


def _row_view(t: Tensor) -> Tensor:
    """``t`` as a matrix whose rows are contiguous (any row stride), copying only if they are not."""
    return t if t.dim() == 2 and t.stride(1) == 1 and t.stride(0) >= t.shape[1] else t.contiguous()


_workspace_bytes_cache: dict = {}


def _conv_workspace(algo: int, num_out: int, K: int, c_in: int, c_out: int, dtype_c: int, out_dtype_c: int,
                    split_k: int, dev: torch.device) -> Optional[Tensor]:
    """Scratch for the offset-sliced tensor-core convolution (None when the launch is one pass)."""
    key = (algo, num_out, K, c_in, c_out, dtype_c, out_dtype_c, split_k, dev.index)
    nbytes = _workspace_bytes_cache.get(key)
    if nbytes is None:
        nbytes = query_bytes("wcn_conv_workspace_bytes", algo, num_out, K, c_in, c_out, dtype_c, out_dtype_c, split_k)
        if len(_workspace_bytes_cache) > 4096:
            _workspace_bytes_cache.clear()
        _workspace_bytes_cache[key] = nbytes
    return torch.empty(nbytes, dtype=torch.uint8, device=dev) if nbytes else None


def sparse_conv_fused(in_features: Tensor, weight: Tensor, kernel_map: IntSearchResult, num_out_coords: int,
                      epilogue: Optional[ConvEpilogue] = None, out_dtype: Optional[torch.dtype] = None,
                      algo: int = CONV_AUTO, tile_order: Optional[bool] = None, split_k: int = 0) -> Tensor:
    """One launch: all kernel offsets + epilogue.  The weight is used in the
    feature dtype (fp32, fp16 or bf16); accumulation is fp32.  ``tile_order`` runs the
    output rows grouped by neighbour pattern (``IntSearchResult.tiled_neighbor_table``;
    same numbers, fewer (tile, offset) pairs to compute); None = by size.  ``split_k``
    (the reference's ``split_k_slices``): 0 lets the library divide the kernel offsets of
    small problems among CTAs, 1 forbids it, 2..16 asks for that many slices.  Features,
    residual and ``epilogue.out`` may be column blocks of wider matrices."""
    require_cuda(in_features, "in_features")
    x = _row_view(in_features)
    if algo == CONV_AUTO and split_k == 0 and not tile_order and num_out_coords > 0:
        # one (input row, offset) pair per output row: the input-side kernel, when it takes the call
        ep0 = epilogue or ConvEpilogue()
        done = None
        if getattr(kernel_map, "_identity", False) and x.shape[0] == num_out_coords:
            dst = None
            if ep0.out_rows is not None and ep0.residual is None and (ep0.out is None or ep0.out.shape[0] == num_out_coords):
                dst = ep0.out_rows.to(device=x.device, dtype=torch.int32).view(1, -1).contiguous()
                ep0 = ConvEpilogue(ep0.scale, ep0.shift, None, ep0.relu, None, ep0.out)
            if ep0.out_rows is None:
                done = sparse_conv_rows_fused(x, weight, dst, num_out_coords, ep0, out_dtype)
        elif getattr(kernel_map, "_one_pair", False) and ep0.out_rows is None and kernel_map._forward is not None:
            done = sparse_conv_rows_fused(x, weight, kernel_map._forward.neighbor_table(x.shape[0]), num_out_coords,
                                          ep0, out_dtype)
        if done is not None:
            return done
    w, packed = _prepared_weight(weight, x.dtype, algo)
    K, c_in, c_out = w.shape
    assert x.shape[1] == c_in, f"features have {x.shape[1]} channels, weight expects {c_in}"
    dev = x.device
    ep = epilogue or ConvEpilogue()
    if ep.out is not None:
        out = ep.out
        out_dtype = out_dtype or out.dtype
        # with out_rows the launch may cover a subset of the rows of a taller destination
        rows_ok = out.shape[0] == num_out_coords or (ep.out_rows is not None and out.shape[0] >= num_out_coords)
        assert out.dtype == out_dtype and out.device == dev and out.dim() == 2 and out.shape[1] == c_out and rows_ok \
            and (out.stride(1) == 1 or num_out_coords == 0), "epilogue.out must be [M, C_out] with contiguous rows"
    else:
        out_dtype = out_dtype or x.dtype
        out = torch.empty((num_out_coords, c_out), dtype=out_dtype, device=dev)
    if num_out_coords == 0:
        return out
    if tile_order is None:
        tile_order = TILE_ORDER_MIN_OFFSETS <= K <= 32 and num_out_coords >= TILE_ORDER_MIN_ROWS
    if tile_order:
        nbr, out_rows = kernel_map.tiled_neighbor_table(num_out_coords)
    else:
        nbr, out_rows = kernel_map.neighbor_table(num_out_coords), None
    assert nbr.shape[0] == K, f"kernel map has {nbr.shape[0]} offsets, weight has {K}"
    if ep.out_rows is not None:
        assert ep.residual is None, "out_rows cannot be combined with a residual"
        assert ep.out_rows.shape == (num_out_coords,), "out_rows must have one entry per output row"
        user_rows = ep.out_rows.to(device=dev, dtype=torch.int32)
        out_rows = user_rows if out_rows is None else user_rows[out_rows.long()]
        out_rows = out_rows.contiguous()
    scale = _as_f32_on(ep.scale, dev)
    shift = _as_f32_on(ep.shift, dev)
    residual = None
    if ep.residual is not None:
        residual = ep.residual if ep.residual.dtype == out_dtype else ep.residual.to(dtype=out_dtype)
        residual = _row_view(residual)
        assert tuple(residual.shape) == (num_out_coords, c_out), \
            f"residual {tuple(residual.shape)} != output {(num_out_coords, c_out)}"
    dc, odc = dtype_code(x.dtype), dtype_code(out_dtype)
    ws = _conv_workspace(algo, num_out_coords, K, c_in, c_out, dc, odc, split_k, dev) if packed is not None else None
    check(lib().wcn_conv_fwd(algo, ptr(x), x.shape[0], x.stride(0), ptr(w), ptr(packed), ptr(nbr), ptr(out_rows),
                             num_out_coords, K, c_in, c_out, dc, ptr(scale), ptr(shift), ptr(residual),
                             residual.stride(0) if residual is not None else 0, int(ep.relu), ptr(out),
                             out.stride(0), odc, split_k, ptr(ws), ws.numel() if ws is not None else 0,
                             ptr(device_status(dev)), stream_ptr(dev)),
          "wcn_conv_fwd")
    if ws is not None:
        LAUNCH_COUNTS["wcn_conv_fwd"] += 1  # the offset-sliced form is two kernels: slices, then their sum + epilogue
    return out


class FusedConvLaunch:
    """One fused convolution with everything that does not change between calls resolved once:
    the weight in the compute dtype and its tensor-core re-tiling, the folded scale / shift vectors
    on the device, the shape and dtype codes, the native entry point.  Calling it enqueues the
    launch with a handful of attribute reads and one foreign call — the per-layer launch record of
    an inference loop (the reference re-derives all of it in Python on every call,
    nn/modules/sequential.py:14-62, nn/functional/sparse_conv.py:1662-1805).

    Arguments are trusted: ``feats`` / ``residual`` / ``out`` are 2-D tensors of the record's dtype
    with contiguous rows on its device (any row stride), ``nbr`` is the ``[K, num_out]`` int32
    neighbour table (tiled, with its ``out_rows``, or plain with ``out_rows=None``)."""

    __slots__ = ("weight", "packed", "scale", "shift", "relu", "K", "c_in", "c_out", "dtype", "device", "_dc",
                 "_w_ptr", "_packed_ptr", "_scale_ptr", "_shift_ptr", "_status_ptr", "_ws_bytes", "_dev_index", "_fn")

    def __init__(self, weight: Tensor, dtype: torch.dtype, scale: Optional[Tensor] = None,
                 shift: Optional[Tensor] = None, relu: bool = False):
        w, packed = _prepared_weight(weight, dtype, CONV_AUTO)
        dev = w.device
        self.weight, self.packed = w, packed
        self.scale, self.shift = _as_f32_on(scale, dev), _as_f32_on(shift, dev)
        self.relu = int(bool(relu))
        self.K, self.c_in, self.c_out = (int(v) for v in w.shape)
        self.dtype, self.device, self._dc = dtype, dev, dtype_code(dtype)
        self._w_ptr, self._packed_ptr = ptr(w), ptr(packed)
        self._scale_ptr, self._shift_ptr = ptr(self.scale), ptr(self.shift)
        self._status_ptr = ptr(device_status(dev))
        self._ws_bytes = {}
        self._dev_index = dev.index if dev.index is not None else torch.cuda.current_device()
        self._fn = lib().wcn_conv_fwd

    def __call__(self, feats: Tensor, nbr: Tensor, out_rows: Optional[Tensor], num_out: int,
                 residual: Optional[Tensor] = None, out: Optional[Tensor] = None) -> Tensor:
        if out is None:
            out = torch.empty((num_out, self.c_out), dtype=self.dtype, device=self.device)
        if num_out == 0:
            return out
        ws = None
        if self._packed_ptr:
            nbytes = self._ws_bytes.get(num_out)
            if nbytes is None:
                nbytes = self._ws_bytes[num_out] = query_bytes("wcn_conv_workspace_bytes", CONV_AUTO, num_out, self.K,
                                                               self.c_in, self.c_out, self._dc, self._dc, 0)
            if nbytes:
                ws = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        rc = self._fn(CONV_AUTO, feats.data_ptr(), feats.shape[0], feats.stride(0), self._w_ptr, self._packed_ptr,
                      nbr.data_ptr(), out_rows.data_ptr() if out_rows is not None else None, num_out, self.K,
                      self.c_in, self.c_out, self._dc, self._scale_ptr, self._shift_ptr,
                      residual.data_ptr() if residual is not None else None,
                      residual.stride(0) if residual is not None else 0, self.relu, out.data_ptr(), out.stride(0),
                      self._dc, 0, ws.data_ptr() if ws is not None else None, nbytes if ws is not None else 0,
                      self._status_ptr, torch._C._cuda_getCurrentRawStream(self._dev_index))
        if rc != 0:
            check(rc, "wcn_conv_fwd")
        if ws is not None:
            LAUNCH_COUNTS["wcn_conv_fwd"] += 1
        return out


def _prepared_rows_weight(weight: Tensor, dtype: torch.dtype):
    """``(packed, c_out_packed)``: the weight re-tiled for the input-side kernel at a width padded to a
    multiple of 16 columns (extra columns zero), or ``(None, 0)`` when that kernel does not take the
    shape.  Cached on the weight tensor like :func:`_prepared_weight`."""
    store = weight.__dict__.setdefault("_wcn_prepared", {})
    hit = store.get((dtype, "rows"))
    if hit is not None and hit[0] == weight._version and hit[3] == weight.device:
        return hit[1], hit[2]
    packed, c_pack = None, 0
    if weight.is_cuda and dtype in (torch.float16, torch.bfloat16):
        K, c_in, c_out = (int(v) for v in weight.shape)
        width = -(-c_out // 16) * 16
        dc = dtype_code(dtype)
        yes = ctypes.c_int32(0)
        check(lib().wcn_conv_rows_supported(K, c_in, width, dc, dc, ctypes.byref(yes)), "wcn_conv_rows_supported")
        if yes.value:
            w = weight.detach().to(dtype=dtype)
            if width != c_out:
                w = torch.nn.functional.pad(w, (0, width - c_out))
            w = w.contiguous()
            nbytes = query_bytes("wcn_conv_packed_weight_bytes", CONV_AUTO, K, c_in, width, dc)
            if nbytes > 0:
                packed, c_pack = torch.empty(nbytes, dtype=torch.uint8, device=w.device), width
                check(lib().wcn_conv_pack_weight(CONV_AUTO, ptr(w), K, c_in, width, dc, ptr(packed), stream_ptr(w.device)),
                      "wcn_conv_pack_weight")
    store[(dtype, "rows")] = (weight._version, packed, c_pack, weight.device)
    return packed, c_pack


def _tma_rows_ok(x: Tensor) -> bool:
    """Rows a tensor map can describe: 16-byte aligned base and row pitch, contiguous rows, at least
    one full 128-row tile."""
    return (x.dim() == 2 and x.shape[0] >= 128 and x.stride(1) == 1 and x.data_ptr() % 16 == 0
            and (x.stride(0) * x.element_size()) % 16 == 0)


def sparse_conv_rows_fused(in_features: Tensor, weight: Tensor, dst_rows: Optional[Tensor], num_out_coords: int,
                           epilogue: Optional[ConvEpilogue] = None,
                           out_dtype: Optional[torch.dtype] = None) -> Optional[Tensor]:
    """A convolution in which every output row has exactly one (input row, offset) pair, run from
    the input side (``wcn_conv_rows_fwd``): ``out[dst_rows[k, j]] = epilogue(in_features[j] @ weight[k])``.
    ``dst_rows`` is int32 ``[K, N_in]`` (entries < 0: no such pair) — for a 2x2x2 stride-2 transposed
    convolution the neighbour table of the matching strided convolution — or None for a 1x1x1
    convolution (``K == 1``, output row = input row).  Returns None when the kernel does not take the
    call (dtype, shape or alignment), so the caller can use the output-side kernels.  Output rows
    that no pair names are left as they were (in a fresh result: uninitialised)."""
    require_cuda(in_features, "in_features")
    x = _row_view(in_features)
    ep = epilogue or ConvEpilogue()
    if x.dtype not in (torch.float16, torch.bfloat16) or not _tma_rows_ok(x) or ep.out_rows is not None:
        return None
    packed, c_pack = _prepared_rows_weight(weight, x.dtype)
    if packed is None:
        return None
    K, c_in, c_out = (int(v) for v in weight.shape)
    assert x.shape[1] == c_in, f"features have {x.shape[1]} channels, weight expects {c_in}"
    dev = x.device
    out_dtype = out_dtype or (ep.out.dtype if ep.out is not None else x.dtype)
    if out_dtype not in (x.dtype, torch.float32):
        return None
    if ep.out is not None:
        out = ep.out
        assert out.dtype == out_dtype and out.device == dev and out.dim() == 2 and out.shape[1] == c_out \
            and out.shape[0] >= num_out_coords and (out.stride(1) == 1 or num_out_coords == 0)
    else:
        out = torch.empty((num_out_coords, c_out), dtype=out_dtype, device=dev)
    if num_out_coords == 0 or x.shape[0] == 0:
        return out
    if dst_rows is not None:
        assert dst_rows.dtype == torch.int32 and tuple(dst_rows.shape) == (K, x.shape[0]) and dst_rows.is_contiguous()
    else:
        assert K == 1 and x.shape[0] == num_out_coords
    residual = None
    if ep.residual is not None:
        residual = ep.residual if ep.residual.dtype == out_dtype else ep.residual.to(dtype=out_dtype)
        residual = _row_view(residual)
        assert tuple(residual.shape) == (num_out_coords, c_out)
    scale, shift = _as_f32_on(ep.scale, dev), _as_f32_on(ep.shift, dev)
    check(lib().wcn_conv_rows_fwd(ptr(x), x.shape[0], x.stride(0), ptr(packed), ptr(dst_rows), num_out_coords, K,
                                  c_in, c_pack, c_out, dtype_code(x.dtype), ptr(scale), ptr(shift), ptr(residual),
                                  residual.stride(0) if residual is not None else 0, int(ep.relu), ptr(out),
                                  out.stride(0), dtype_code(out_dtype), ptr(device_status(dev)), stream_ptr(dev)),
          "wcn_conv_rows_fwd")
    return out


class FusedRowsLaunch:
    """The launch record of a one-pair-per-output-row convolution (:func:`sparse_conv_rows_fused`) with
    everything constant resolved once, as :class:`FusedConvLaunch` is for the output-side kernels.
    ``usable`` is False when the input-side kernel does not take the layer's shape."""

    __slots__ = ("packed", "scale", "shift", "relu", "K", "c_in", "c_out", "c_pack", "dtype", "device", "_dc",
                 "_packed_ptr", "_scale_ptr", "_shift_ptr", "_status_ptr", "_dev_index", "_fn", "usable")

    def __init__(self, weight: Tensor, dtype: torch.dtype, scale: Optional[Tensor] = None,
                 shift: Optional[Tensor] = None, relu: bool = False):
        self.packed, self.c_pack = _prepared_rows_weight(weight, dtype)
        self.usable = self.packed is not None
        dev = weight.device
        self.scale, self.shift = _as_f32_on(scale, dev), _as_f32_on(shift, dev)
        self.relu = int(bool(relu))
        self.K, self.c_in, self.c_out = (int(v) for v in weight.shape)
        self.dtype, self.device = dtype, dev
        self._dc = dtype_code(dtype) if self.usable else 0
        self._packed_ptr = ptr(self.packed)
        self._scale_ptr, self._shift_ptr = ptr(self.scale), ptr(self.shift)
        self._status_ptr = ptr(device_status(dev)) if self.usable else None
        self._dev_index = dev.index if dev.index is not None else (torch.cuda.current_device() if self.usable else 0)
        self._fn = lib().wcn_conv_rows_fwd

    def takes(self, feats: Tensor) -> bool:
        return self.usable and _tma_rows_ok(feats)

    def __call__(self, feats: Tensor, dst_rows: Optional[Tensor], num_out: int, residual: Optional[Tensor] = None,
                 out: Optional[Tensor] = None) -> Tensor:
        if out is None:
            out = torch.empty((num_out, self.c_out), dtype=self.dtype, device=self.device)
        if num_out == 0 or feats.shape[0] == 0:
            return out
        rc = self._fn(feats.data_ptr(), feats.shape[0], feats.stride(0), self._packed_ptr,
                      dst_rows.data_ptr() if dst_rows is not None else None, num_out, self.K, self.c_in, self.c_pack,
                      self.c_out, self._dc, self._scale_ptr, self._shift_ptr,
                      residual.data_ptr() if residual is not None else None,
                      residual.stride(0) if residual is not None else 0, self.relu, out.data_ptr(), out.stride(0),
                      self._dc, self._status_ptr, torch._C._cuda_getCurrentRawStream(self._dev_index))
        if rc != 0:
            check(rc, "wcn_conv_rows_fwd")
        return out


def _implicit_gemm_forward_logic(in_features: Tensor, weight: Tensor, kernel_map: IntSearchResult,
                                 num_out_coords: int, compute_dtype: Optional[torch.dtype],
                                 fwd_block_size: Optional[int] = None,
                                 epilogue: Optional[ConvEpilogue] = None) -> Tensor:
    """Both operands are cast to the lower-ranked of (feature/compute dtype,
    weight dtype); the result returns in the feature dtype (reference :358-415,
    :495-544).  ``fwd_block_size`` is accepted and ignored (no tunables)."""
    feature_dtype = compute_dtype if compute_dtype is not None else in_features.dtype
    min_dtype = _min_dtype(feature_dtype, weight.dtype)
    if min_dtype == torch.float64:
        raise ValueError("float64 is not supported by the native kernels; use explicit_gemm")
    x = in_features if in_features.dtype == min_dtype else in_features.to(dtype=min_dtype)
    if x.requires_grad:
        x = x.detach()
    return sparse_conv_fused(x, weight, kernel_map, num_out_coords, epilogue, out_dtype=in_features.dtype
                             if in_features.dtype in (torch.float32, torch.float16, torch.bfloat16) else None)


_cutlass_implicit_gemm_forward_logic = _implicit_gemm_forward_logic


# --------------------------------------------------------------------------- output coordinates + kernel map


def _with_z(bcoords: Tensor) -> Tensor:
    """(batch, x, y) rows as (batch, x, y, 0): a 2-D grid is the z = 0 slab of a 3-D one, and a
    kx x ky window on it is a kx x ky x 1 window, in the same offset order."""
    return torch.cat([bcoords, torch.zeros((bcoords.shape[0], 1), dtype=bcoords.dtype, device=bcoords.device)], dim=1)


def _generate_kernel_map_nd(in_coords: Tensor, out_coords: Tensor, stride, kernel_size, kernel_dilation,
                            hashtable=None, bricks=None) -> IntSearchResult:
    """``generate_kernel_map`` for 3 spatial dimensions as is, for 2 through the z = 0 slab."""
    if in_coords.shape[1] == 4:
        return generate_kernel_map(in_coords, out_coords, stride, kernel_size, kernel_dilation, hashtable=hashtable,
                                   bricks=bricks)
    assert in_coords.shape[1] == 3 and out_coords.shape[1] == 3, "coordinates must have 2 or 3 spatial dimensions"
    same = out_coords.data_ptr() == in_coords.data_ptr() and out_coords.shape == in_coords.shape
    in4 = _with_z(in_coords)
    out4 = in4 if same else _with_z(out_coords)
    return generate_kernel_map(in4, out4, tuple(stride) + (1,), tuple(kernel_size) + (1,),
                               tuple(kernel_dilation) + (1,))


def generate_output_coords_and_kernel_map(input_sparse_tensor: Voxels, kernel_size: Tuple[int, ...],
                                          kernel_dilation: Tuple[int, ...], stride: Tuple[int, ...],
                                          generative: bool, transposed: bool,
                                          output_spatially_sparse_tensor: Optional[Voxels],
                                          stride_mode: STRIDED_CONV_MODE = STRIDED_CONV_MODE.STRIDE_ONLY,
                                          order: POINT_ORDERING = POINT_ORDERING.RANDOM):
    """(batch-indexed output coords, output offsets, kernel map); maps are cached on
    the input's shared cache and a transposed map reuses the forward one."""
    if stride_mode != STRIDED_CONV_MODE.STRIDE_ONLY and any(s != 1 for s in stride):
        raise ValueError("with stride_mode=reduce_and_stride the caller pools first and passes stride 1")
    in_coords = input_sparse_tensor.batch_indexed_coordinates
    if in_coords.dtype != torch.int32:
        in_coords = in_coords.to(torch.int32)

    if output_spatially_sparse_tensor is not None:
        assert not generative, "Output spatially sparse tensor is not supported with generative convolution"
        out_coords = output_spatially_sparse_tensor.batch_indexed_coordinates
        if out_coords.dtype != torch.int32:
            out_coords = out_coords.to(torch.int32)
        out_offsets = output_spatially_sparse_tensor.offsets
    elif any(s != 1 for s in stride):
        down = strided_coordinates(input_sparse_tensor.batched_coordinates, stride)
        if generative:  # the strided set grown by the kernel window (reference :1861-1866)
            down = expanded_coordinates(down, kernel_size, kernel_dilation)
        out_coords, out_offsets = down.batch_indexed_coordinates, down.offsets
    elif generative:
        assert not transposed, "Transposed and generative convolution is not supported yet"
        if in_coords.shape[1] != 4:
            raise NotImplementedError("generative convolution needs 3 spatial dimensions")
        grown = expanded_coordinates(input_sparse_tensor.batched_coordinates, kernel_size, kernel_dilation)
        out_coords, out_offsets = grown.batch_indexed_coordinates, grown.offsets
    else:
        out_coords, out_offsets = in_coords, input_sparse_tensor.offsets

    if order != POINT_ORDERING.RANDOM:
        perm = encode(out_coords[:, 1:], batch_offsets=out_offsets, order=order, return_perm=True).perm
        out_coords = out_coords[perm]

    def key_for(transposed_, in_off, out_off):
        return IntSearchCacheKey(kernel_size=kernel_size, kernel_dilation=kernel_dilation, transposed=transposed_,
                                 generative=generative, stride_mode=str(stride_mode),
                                 skip_symmetric_kernel_map=False, in_offsets=in_off, out_offsets=out_off)

    key = key_for(transposed, input_sparse_tensor.offsets, out_offsets)
    cache = input_sparse_tensor.cache
    if cache is not None:
        hit = cache.get(key)
        if hit is not None:
            return out_coords, out_offsets, hit

    if transposed:
        fwd = None
        if cache is not None:
            fwd = cache.get(key_for(False, out_offsets, input_sparse_tensor.offsets))
        if fwd is None:
            # forward map: table on the (fine) output coordinates, (coarse) inputs * stride as queries
            fwd = _generate_kernel_map_nd(out_coords, in_coords, stride, kernel_size, kernel_dilation,
                                          hashtable=_cached_table(output_spatially_sparse_tensor, out_coords),
                                          bricks=_cached_bricks(output_spatially_sparse_tensor, out_coords))
        kernel_map = fwd.swapped(num_in=out_coords.shape[0])
        # Window = stride without dilation, and the inputs are exactly the strided outputs: every output
        # voxel then has one parent and one offset, which the input-side kernel exploits.
        fine = output_spatially_sparse_tensor.batched_coordinates if output_spatially_sparse_tensor is not None else None
        parent = fine._shared.get(("strided", tuple(int(s) for s in stride))) if fine is not None else None
        kernel_map._one_pair = (tuple(kernel_size) == tuple(stride) and all(int(d) == 1 for d in kernel_dilation)
                                and parent is not None
                                and parent._shared is input_sparse_tensor.batched_coordinates._shared)
    else:
        kernel_map = _generate_kernel_map_nd(in_coords, out_coords, stride, kernel_size, kernel_dilation,
                                             hashtable=_cached_table(input_sparse_tensor, in_coords),
                                             bricks=_cached_bricks(input_sparse_tensor, in_coords))

    if input_sparse_tensor.cache is None:
        input_sparse_tensor._extra_attributes["_cache"] = IntSearchCache()
    input_sparse_tensor.cache.put(key, kernel_map)
    return out_coords, out_offsets, kernel_map


def strided_coordinates(coords: IntCoords, stride: Tuple[int, ...]) -> IntCoords:
    """The distinct rows of ``floor(coords / stride)`` as an ``IntCoords`` that already knows its
    batch-indexed form.  Computed once per (coordinate set, stride) and kept with the
    coordinate set, so that every layer striding the same coordinates shares one result and
    :func:`prefetch_strided_coordinates` can compute a whole pyramid ahead of the features."""
    stride = tuple(int(s) for s in stride)
    key = ("strided", stride)
    hit = coords._shared.get(key)
    if hit is None:
        bc = coords.batch_indexed_coordinates
        if bc.dtype != torch.int32:
            bc = bc.to(torch.int32)
        if bc.shape[1] == 3:  # two spatial dimensions: stride the z = 0 slab, then drop z again
            out4, out_offsets = stride_coords(_with_z(bc), stride + (1,), in_offsets=coords.offsets)
            out_coords = out4[:, :3].contiguous()
        else:
            out_coords, out_offsets = stride_coords(bc, stride, in_offsets=coords.offsets)
        hit = IntCoords(out_coords[:, 1:], offsets=out_offsets)
        hit._bcoords = out_coords
        origin = coords.morton_origin
        if origin is not None and bc.shape[1] == 4:
            # First occurrences of floor(c / s) in Morton order are themselves in Morton order about
            # floor(origin / s) whenever the origin is a multiple of the stride; the brick table's build
            # checks the order on the device, so a misaligned origin only costs the fallback search.
            s_t = stride[0] if len(set(stride)) == 1 else torch.tensor(stride, dtype=torch.int32, device=origin.device)
            hit.morton_origin = torch.div(origin, s_t, rounding_mode="floor").to(torch.int32)
        coords._shared[key] = hit
    return hit


def expanded_coordinates(coords: IntCoords, kernel_size: Tuple[int, ...], kernel_dilation: Tuple[int, ...]) -> IntCoords:
    """The coordinates a kernel window reaches from ``coords`` (the output support of a generative
    convolution), computed once per (coordinate set, window) and kept with the coordinate set."""
    key = ("expanded", tuple(int(k) for k in kernel_size), tuple(int(d) for d in kernel_dilation))
    hit = coords._shared.get(key)
    if hit is None:
        bc = coords.batch_indexed_coordinates
        rows, offsets = expand_coords(bc if bc.dtype == torch.int32 else bc.to(torch.int32), key[1], key[2])
        hit = IntCoords(rows[:, 1:], offsets=offsets, tensor_stride=coords.tensor_stride)
        hit._bcoords = rows
        coords._shared[key] = hit
    return hit


def prefetch_strided_coordinates(voxels: Voxels, strides) -> List[IntCoords]:
    """Compute the coordinate pyramid ``voxels -> /strides[0] -> /strides[1] ...`` now.

    Sizing each strided coordinate set costs one host synchronisation.  Done lazily inside the
    strided convolutions, each of those waits for every feature kernel queued before it; done
    here, before the first convolution is queued, the waits only cover the small coordinate
    kernels and the whole network can then be queued without the host ever waiting.  (An
    addition to the reference surface; results are identical with or without the call.)"""
    nd = voxels.num_spatial_dims
    level = voxels.batched_coordinates
    steps = [ntuple(s, ndim=nd) for s in strides]
    bc = level.batch_indexed_coordinates
    if (nd == 3 and bc.is_cuda and bc.dtype == torch.int32 and 0 < bc.shape[0] <= PYRAMID_ONE_SYNC_MAX_ROWS
            and steps and ("strided", steps[0]) not in level._shared):
        _pyramid_in_one_sync(level, steps)
    out = []
    for s in steps:
        level = strided_coordinates(level, s)
        out.append(level)
    return out


# Below this many rows the whole coordinate pyramid is computed from the finest level with a single
# host synchronisation (every level hashes all the fine rows); above it the levels are chained
# (each hashes only the rows of the level before it, one synchronisation per level).
PYRAMID_ONE_SYNC_MAX_ROWS = 700_000


def _pyramid_in_one_sync(level: IntCoords, steps) -> None:
    """Fill the ``strided`` entries of ``level`` and of every coarser level it leads to, so that the
    ``strided_coordinates`` calls that follow find them."""
    from ...geometry.coords.ops.stride import strided_pyramid
    totals, acc = [], (1, 1, 1)
    for s in steps:
        acc = tuple(a * b for a, b in zip(acc, s))
        totals.append(acc)
    results = strided_pyramid(level.batch_indexed_coordinates, totals, level.offsets)
    origin = level.morton_origin
    for s, total, (rows, offsets) in zip(steps, totals, results):
        hit = IntCoords(rows[:, 1:], offsets=offsets)
        hit._bcoords = rows
        if origin is not None:
            t = total[0] if len(set(total)) == 1 else torch.tensor(total, dtype=torch.int32, device=origin.device)
            hit.morton_origin = torch.div(origin, t, rounding_mode="floor").to(torch.int32)
        level._shared[("strided", s)] = hit
        level = hit


def _cached_table(voxels: Optional[Voxels], coords: Tensor):
    """The hash table of a tensor's own coordinates (built once per coordinate set and shared
    by every layer that searches it), or None when ``coords`` is not that tensor's own array."""
    if voxels is None or coords.shape[1] != 4:
        return None
    ic = voxels.batched_coordinates
    own = ic.batch_indexed_coordinates
    if own.dtype != torch.int32 or own.data_ptr() != coords.data_ptr() or own.shape != coords.shape:
        return None
    return ic.hashmap


def _cached_bricks(voxels: Optional[Voxels], coords: Tensor):
    """The brick table of a tensor's own Morton-ordered coordinates (None when they are not)."""
    if _cached_table(voxels, coords) is None:
        return None
    return voxels.batched_coordinates.bricks


# --------------------------------------------------------------------------- autograd


def sparse_conv_wgrad(in_features: Tensor, grad_output: Tensor, kernel_map: IntSearchResult,
                      num_out_coords: int, tile_order: bool = False) -> Optional[Tensor]:
    """``dW[k] = X[in_k]^T @ dY[out_k]`` for every kernel offset in one launch on the tensor cores
    (fp16 / bf16 operands, fp32 result ``[K, C_in, C_out]``), or None when the shape is not one the
    native kernel takes (the caller then uses a GEMM per offset)."""
    require_cuda(in_features, "in_features")
    x, g = in_features.contiguous(), grad_output.contiguous()
    K, c_in, c_out = len(kernel_map), x.shape[1], g.shape[1]
    if (x.dtype not in (torch.float16, torch.bfloat16) or g.dtype != x.dtype or c_in % 32 or c_out % 32
            or c_out > 256 or K > 32 or x.shape[0] == 0 or num_out_coords == 0):
        return None
    dev = x.device
    tiled = bool(tile_order)
    if tiled:
        nbr, out_rows = kernel_map.tiled_neighbor_table(num_out_coords)
    else:
        nbr, out_rows = kernel_map.neighbor_table(num_out_coords), None
    masks = kernel_map.tile_masks(num_out_coords, tiled) if K > 1 else None  # steps without neighbours are skipped
    gw = torch.zeros((K, c_in, c_out), dtype=torch.float32, device=dev)
    check(lib().wcn_conv_wgrad(ptr(x), x.shape[0], ptr(g), ptr(nbr), ptr(out_rows), ptr(masks), num_out_coords, K,
                               c_in, c_out,
                               dtype_code(x.dtype), ptr(gw), ptr(device_status(dev)), stream_ptr(dev)),
          "wcn_conv_wgrad")
    return gw


def _normalize_bwd_algo(algo) -> SPARSE_CONV_BWD_ALGO_MODE:
    """Enum | str | list of either -> one algorithm; with a list the first native entry wins
    (no tuner), as for the forward algorithm."""
    items = list(algo) if isinstance(algo, (list, tuple)) else [algo]
    items = [SPARSE_CONV_BWD_ALGO_MODE(a.lower()) if isinstance(a, str) else a for a in items]
    for a in items:
        if a != SPARSE_CONV_BWD_ALGO_MODE.EXPLICIT_GEMM:
            return a
    return items[0]


class _SparseConvFunction(torch.autograd.Function):
    """Forward through the native kernels.  Backward with the explicit algorithm: the reference's
    formulas on the compact map (:314-355), dX[in_k] += dY[out_k] @ W_k^T and
    dW_k = X[in_k]^T @ dY[out_k], a GEMM per offset.  With the implicit algorithms (the reference's
    AD gather-scatter with the maps swapped and W^T, and its trAB gather / split-K kernels,
    :472-480, 591-604): dX is ONE launch of the forward kernel over the transposed neighbour table
    with the weights transposed, dW ONE launch of the tensor-core weight-gradient kernel (shapes it
    does not take fall back to the per-offset GEMMs)."""

    @staticmethod
    def forward(ctx, in_features, weight, kernel_map, num_out_coords, algo, compute_dtype, epilogue,
                bwd_algo=SPARSE_CONV_BWD_ALGO_MODE.EXPLICIT_GEMM):
        ctx.kernel_map = kernel_map
        ctx.compute_dtype = compute_dtype
        ctx.bwd_algo = bwd_algo
        ctx.save_for_backward(in_features, weight)
        if algo == SPARSE_CONV_FWD_ALGO_MODE.EXPLICIT_GEMM:
            return _explicit_gemm_forward_logic(in_features, weight, kernel_map, num_out_coords, compute_dtype)
        return _implicit_gemm_forward_logic(in_features, weight, kernel_map, num_out_coords, compute_dtype,
                                            epilogue=epilogue)

    @staticmethod
    def backward(ctx, grad_output):
        x, w = ctx.saved_tensors
        km = ctx.kernel_map
        dt = ctx.compute_dtype if ctx.compute_dtype is not None else x.dtype
        xc, wc, gc = x.to(dt), w.to(dt), grad_output.contiguous().to(dt)
        need_gx, need_gw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        native_dx = (need_gx and ctx.bwd_algo != SPARSE_CONV_BWD_ALGO_MODE.EXPLICIT_GEMM and gc.is_cuda
                     and dt in (torch.float32, torch.float16, torch.bfloat16) and x.shape[0] > 0)
        gx = None
        if native_dx:
            with torch.no_grad():
                wt = wc.detach().transpose(1, 2).contiguous()  # [K, C_out, C_in]
                gx = sparse_conv_fused(gc.detach(), wt, km.swapped(num_in=x.shape[0]), x.shape[0])
        elif need_gx:
            gx = torch.zeros_like(xc)
        gw = None
        if need_gw and native_dx:  # the implicit algorithms: one tensor-core launch when the shape allows
            with torch.no_grad():
                gw = sparse_conv_wgrad(xc.detach(), gc.detach(), km, gc.shape[0])
        native_dw = gw is not None
        if need_gw and not native_dw:
            gw = torch.zeros_like(wc)
        need_gw = need_gw and not native_dw
        if need_gw or (need_gx and not native_dx):
            offsets, in_maps, out_maps = km.offsets, km.in_maps, km.out_maps
            for k in range(len(km)):
                s, e = int(offsets[k]), int(offsets[k + 1])
                if e == s:
                    continue
                go = _gather_rows(gc, out_maps[s:e])
                if need_gx and not native_dx:
                    _scatter_add_rows(torch.matmul(go, wc[k].T), in_maps[s:e], gx)
                if need_gw:
                    gw[k] = torch.matmul(_gather_rows(xc, in_maps[s:e]).T, go)
        return (gx.to(x.dtype) if gx is not None else None, gw.to(w.dtype) if gw is not None else None,
                None, None, None, None, None, None)


# --------------------------------------------------------------------------- entry point


def spatially_sparse_conv(
    input_sparse_tensor: Voxels,
    weight: Tensor,
    kernel_size: Union[int, List[int], Tuple[int, ...]],
    stride: Union[int, List[int], Tuple[int, ...]] = 1,
    kernel_dilation: Union[int, List[int], Tuple[int, ...]] = 1,
    bias: Optional[Tensor] = None,
    kernel_matmul_batch_size: int = 2,
    generative: bool = False,
    output_spatially_sparse_tensor: Optional[Voxels] = None,
    transposed: bool = False,
    fwd_algo: Union[SPARSE_CONV_FWD_ALGO_MODE, List[SPARSE_CONV_FWD_ALGO_MODE]] = SPARSE_CONV_FWD_ALGO_MODE.EXPLICIT_GEMM,
    bwd_algo: Union[SPARSE_CONV_BWD_ALGO_MODE, List[SPARSE_CONV_BWD_ALGO_MODE]] = SPARSE_CONV_BWD_ALGO_MODE.EXPLICIT_GEMM,
    stride_mode: STRIDED_CONV_MODE = STRIDED_CONV_MODE.STRIDE_ONLY,
    stride_reduce: str = "max",
    order: POINT_ORDERING = POINT_ORDERING.RANDOM,
    compute_dtype: Optional[torch.dtype] = None,
    implicit_matmul_fwd_block_size: Optional[int] = 16,
    implicit_matmul_bwd_block_size: Optional[int] = 16,
    epilogue: Optional[ConvEpilogue] = None,
) -> Voxels:
    """Sparse convolution of a ``Voxels`` tensor with ``weight [K, C_in, C_out]``.

    ``epilogue`` (an addition to the reference signature) fuses scale/shift,
    residual add and ReLU into the kernel; it forces the native implicit kernel.
    """
    if not isinstance(input_sparse_tensor, Voxels):
        raise TypeError("Native spatially_sparse_conv expects input_sparse_tensor of type Voxels, got "
                        f"{type(input_sparse_tensor)}")
    if output_spatially_sparse_tensor is not None and not isinstance(output_spatially_sparse_tensor, Voxels):
        raise TypeError("Native spatially_sparse_conv expects output_spatially_sparse_tensor of type Voxels or "
                        f"None, got {type(output_spatially_sparse_tensor)}")
    nd = input_sparse_tensor.num_spatial_dims
    _kernel_size = ntuple(kernel_size, ndim=nd)
    _kernel_dilation = ntuple(kernel_dilation, ndim=nd)
    _stride = ntuple(stride, ndim=nd)
    algo = _normalize_fwd_algo(fwd_algo)
    feats = input_sparse_tensor.feature_tensor
    # a trainable bias counts: it must reach autograd as a tensor, never folded into a detached epilogue
    needs_grad = torch.is_grad_enabled() and (feats.requires_grad or weight.requires_grad
                                              or (bias is not None and bias.requires_grad))

    if all(k == 1 for k in _kernel_size) and all(s == 1 for s in _stride):
        native = feats.is_cuda and feats.dtype in (torch.float32, torch.float16, torch.bfloat16)
        if epilogue is None and (needs_grad or not native):
            out = feats @ weight[0].to(feats.dtype) if weight.dtype != feats.dtype else feats @ weight[0]
            if bias is not None:
                out = out + bias.to(out.dtype)
            return input_sparse_tensor.replace(batched_features=out)
        # 1x1x1 in inference: the native kernel over the identity neighbour table, bias and any fused
        # tail in its epilogue
        n = feats.shape[0]
        ident = _identity_map(n, feats.device)
        ep = _merge_bias(epilogue, bias)
        out = _implicit_gemm_forward_logic(feats, weight, ident, n, compute_dtype, epilogue=ep)
        return input_sparse_tensor._derive(out)

    in_tensor_stride = input_sparse_tensor.tensor_stride
    if in_tensor_stride is None:
        in_tensor_stride = ntuple(1, ndim=nd)
    if transposed and not generative:
        assert output_spatially_sparse_tensor is not None, \
            "Output spatially sparse tensor is required for transposed convolution"
    if not transposed:
        out_tensor_stride = tuple(o * s for o, s in zip(_stride, in_tensor_stride))
    else:
        if output_spatially_sparse_tensor is not None and output_spatially_sparse_tensor.tensor_stride is not None:
            out_tensor_stride = output_spatially_sparse_tensor.tensor_stride
        else:
            out_tensor_stride = ntuple(1, ndim=nd)
        assert any(o < i for o, i in zip(out_tensor_stride, in_tensor_stride)), \
            "Output stride is larger than input stride"

    if stride_mode == STRIDED_CONV_MODE.REDUCE_AND_STRIDE and any(s != 1 for s in _stride) and not transposed:
        # pool the stride window first, then convolve at stride 1 on the pooled tensor (:1753-1767)
        from .sparse_pool import sparse_reduce
        input_sparse_tensor = sparse_reduce(input_sparse_tensor, kernel_size=_stride, stride=_stride,
                                            reduction=stride_reduce)
        feats = input_sparse_tensor.feature_tensor
        _stride = ntuple(1, ndim=nd)

    effective_compute_dtype = compute_dtype if compute_dtype is not None else feats.dtype

    out_coords, out_offsets, kernel_map = generate_output_coords_and_kernel_map(
        input_sparse_tensor=input_sparse_tensor, kernel_size=_kernel_size, kernel_dilation=_kernel_dilation,
        stride=_stride, generative=generative, transposed=transposed,
        output_spatially_sparse_tensor=output_spatially_sparse_tensor, stride_mode=stride_mode, order=order)
    num_out = out_coords.shape[0]

    if algo == SPARSE_CONV_FWD_ALGO_MODE.EXPLICIT_GEMM and epilogue is None:
        if needs_grad:
            out = _SparseConvFunction.apply(feats, weight, kernel_map, num_out, algo, effective_compute_dtype, None,
                                            _normalize_bwd_algo(bwd_algo))
        else:
            out = _explicit_gemm_forward_logic(feats, weight, kernel_map, num_out, effective_compute_dtype)
        if bias is not None:
            out = out + bias.to(out.dtype)
    else:
        if needs_grad:
            if epilogue is not None:
                raise RuntimeError("a fused epilogue is an inference feature; run under torch.no_grad()")
            # the bias is added outside the Function, where autograd sees it (reference :1794-1795)
            out = _SparseConvFunction.apply(feats, weight, kernel_map, num_out,
                                            SPARSE_CONV_FWD_ALGO_MODE.IMPLICIT_GEMM, effective_compute_dtype, None,
                                            _normalize_bwd_algo(bwd_algo))
            if bias is not None:
                out = out + bias.to(out.dtype)
        else:
            out = _implicit_gemm_forward_logic(feats, weight, kernel_map, num_out, effective_compute_dtype,
                                               epilogue=_merge_bias(epilogue, bias))

    # Output coordinates: the input's own coordinate object when they are unchanged, the target's for
    # a transposed convolution, the cached strided set otherwise; all of them already know their
    # batch-indexed form and hash table, so nothing is rebuilt layer after layer.
    if order == POINT_ORDERING.RANDOM:
        own = False
        if output_spatially_sparse_tensor is not None:
            out_ic = output_spatially_sparse_tensor.batched_coordinates
        elif all(s == 1 for s in _stride):
            out_ic = input_sparse_tensor.batched_coordinates
        else:
            out_ic, own = strided_coordinates(input_sparse_tensor.batched_coordinates, _stride), True
        if generative:
            out_ic, own = expanded_coordinates(out_ic, _kernel_size, _kernel_dilation), True
        if out_ic.tensor_stride != out_tensor_stride:
            if own and out_ic.tensor_stride is None:
                out_ic.tensor_stride = out_tensor_stride  # the cached set is labelled once
            else:  # same rows under another stride label: a view that shares the derived data
                out_ic = IntCoords(out_ic.batched_tensor, offsets=out_ic.offsets,
                                   tensor_stride=out_tensor_stride).share_derived(out_ic)
        return input_sparse_tensor._derive(out, out_ic)
    out_ic = IntCoords(out_coords[:, 1:], offsets=out_offsets if out_offsets.device.type == "cpu" else out_offsets.cpu())
    out_ic._bcoords = out_coords
    return input_sparse_tensor.replace(batched_coordinates=out_ic, batched_features=out,
                                       tensor_stride=out_tensor_stride)


def _merge_bias(epilogue: Optional[ConvEpilogue], bias: Optional[Tensor]) -> Optional[ConvEpilogue]:
    """The reference adds the bias right after the convolution (:1794-1795), i.e.
    before any BatchNorm that follows: (conv + b) * scale + shift
    = conv * scale + (shift + b * scale)."""
    if bias is None:
        return epilogue
    b = bias.detach().float()
    if epilogue is None:
        return ConvEpilogue(shift=b)
    if epilogue.scale is None and epilogue.shift is None:
        return ConvEpilogue(shift=b, residual=epilogue.residual, relu=epilogue.relu, out_rows=epilogue.out_rows,
                            out=epilogue.out)
    if epilogue.scale is not None:
        b = b * epilogue.scale.to(b.device).float()
    shift = b if epilogue.shift is None else epilogue.shift.to(b.device).float() + b
    return ConvEpilogue(scale=epilogue.scale, shift=shift, residual=epilogue.residual, relu=epilogue.relu,
                        out_rows=epilogue.out_rows, out=epilogue.out)


_identity_maps: dict = {}


def _identity_map(n: int, device: torch.device) -> IntSearchResult:
    """Neighbour table of a 1x1x1 convolution: row m reads row m."""
    key = (n, str(device))
    hit = _identity_maps.get(key)
    if hit is None:
        nbr = torch.arange(n, dtype=torch.int32, device=device).unsqueeze(0).contiguous()
        hit = IntSearchResult.from_neighbor_table(nbr, n, None, 0)
        hit._identity = True
        if len(_identity_maps) > 64:
            _identity_maps.clear()
        _identity_maps[key] = hit
    return hit
