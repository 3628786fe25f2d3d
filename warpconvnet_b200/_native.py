"""ctypes binding of ``csrc/libwcn_b200.so`` (declared in ``include/wcn_b200.h``).

The library is the only compute back-end of this package: when it is missing
or cannot be loaded, every operation raises; there is no CPU or eager fallback.
PyTorch is used for device memory and streams only.
"""
from __future__ import annotations

import ctypes
import os
from collections import Counter
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "libwcn_b200.so")

WCN_F32, WCN_F16, WCN_BF16 = 0, 1, 2
CONV_AUTO, CONV_SIMT, CONV_TCGEN05 = 0, 1, 2
_DTYPE_CODE = {torch.float32: WCN_F32, torch.float16: WCN_F16, torch.bfloat16: WCN_BF16}

_c_i32, _c_i64, _c_vp = ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p
_p_i64 = ctypes.POINTER(ctypes.c_int64)

# name -> argument types, exactly the prototypes of include/wcn_b200.h
SIGNATURES = {
    "wcn_version": [],
    "wcn_hash_table_bytes": [_c_i64, _p_i64],
    "wcn_hash_build": [_c_vp, _c_i64, _c_vp, _c_vp, _c_i64, _c_i32, _c_vp, _c_vp, _c_vp],
    "wcn_hash_search": [_c_vp, _c_i64, _c_i32, _c_vp, _c_i64, _c_vp, _c_vp],
    "wcn_unique_workspace_bytes": [_c_i64, _p_i64],
    "wcn_unique_mark": [_c_vp, _c_i64, _c_vp, _c_vp, _c_i64, _c_i32, _c_vp, _c_vp, _c_vp],
    "wcn_unique_emit": [_c_vp, _c_i64, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp],
    "wcn_kmap_workspace_bytes": [_c_i64, _c_i32, _p_i64],
    "wcn_kmap_search": [_c_vp, _c_i64, _c_i32, _c_vp, _c_i64, _c_vp, _c_vp, _c_i32, _c_vp, _c_vp, _c_vp],
    "wcn_kmap_search_static": [_c_vp, _c_i64, _c_i32, _c_vp, _c_i64, _c_vp, _c_vp, _c_i32, _c_vp, _c_vp, _c_vp],
    "wcn_kmap_search_self": [_c_vp, _c_i64, _c_i32, _c_vp, _c_i64, _c_vp, _c_vp, _c_vp, _c_vp],
    "wcn_kmap_search_dilated": [_c_vp, _c_i64, _c_i32, _c_vp, _c_i64, _c_vp, _c_vp, _c_vp, _c_vp, _c_i32, _c_vp, _c_vp, _c_vp],
    "wcn_kmap_count": [_c_vp, _c_i64, _c_i32, _c_vp, _c_vp],
    "wcn_brick_table_bytes": [_c_i64, _p_i64],
    "wcn_brick_build": [_c_vp, _c_i64, _c_vp, _c_vp, _c_vp],
    "wcn_kmap_search_bricks": [_c_vp, _c_vp, _c_i64, _c_i32, _c_vp, _c_i64, _c_vp, _c_vp, _c_vp, _c_vp],
    "wcn_kmap_scan": [_c_vp, _c_i64, _c_i32, _c_vp, _c_vp],
    "wcn_kmap_compact": [_c_vp, _c_i64, _c_i32, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp],
    "wcn_nbr_from_maps": [_c_vp, _c_vp, _c_vp, _c_i32, _c_i64, _c_i64, _c_vp, _c_vp],
    "wcn_nbr_transpose": [_c_vp, _c_i32, _c_i64, _c_i64, _c_vp, _c_vp],
    "wcn_morton20": [_c_vp, _c_i64, _c_i32, _c_i32, _c_vp, _c_vp, _c_vp],
    "wcn_gather_rows": [_c_vp, _c_i64, _c_vp, _c_vp, _c_i64, _c_i32, _c_i32, _c_vp, _c_vp],
    "wcn_scatter_add_rows": [_c_vp, _c_vp, _c_vp, _c_i64, _c_i64, _c_i32, _c_i32, _c_vp, _c_vp],
    "wcn_conv_packed_weight_bytes": [_c_i32, _c_i32, _c_i32, _c_i32, _c_i32, _p_i64],
    "wcn_conv_pack_weight": [_c_i32, _c_vp, _c_i32, _c_i32, _c_i32, _c_i32, _c_vp, _c_vp],
    "wcn_kmap_tile_order": [_c_vp, _c_i64, _c_i32, _c_vp, _c_vp, _c_vp],
    "wcn_row_reduce": [_c_vp, _c_i64, _c_vp, _c_i64, _c_i32, _c_i32, _c_i32, _c_i32, _c_vp, _c_vp, _c_vp],
    "wcn_kmap_tile_masks": [_c_vp, _c_i64, _c_i32, _c_vp, _c_vp],
    "wcn_conv_wgrad": [_c_vp, _c_i64, _c_vp, _c_vp, _c_vp, _c_vp, _c_i64, _c_i32, _c_i32, _c_i32, _c_i32, _c_vp, _c_vp, _c_vp],
    "wcn_conv_workspace_bytes": [_c_i32, _c_i64, _c_i32, _c_i32, _c_i32, _c_i32, _c_i32, _c_i32, _p_i64],
    "wcn_conv_fwd": [_c_i32, _c_vp, _c_i64, _c_i64, _c_vp, _c_vp, _c_vp, _c_vp, _c_i64, _c_i32, _c_i32, _c_i32, _c_i32,
                     _c_vp, _c_vp, _c_vp, _c_i64, _c_i32, _c_vp, _c_i64, _c_i32, _c_i32, _c_vp, _c_i64, _c_vp, _c_vp],
    "wcn_selftest_bounded_wait": [_c_i64, _c_vp, _c_vp, _c_vp],
    "wcn_conv_rows_supported": [_c_i32, _c_i32, _c_i32, _c_i32, _c_i32, _c_vp],
    "wcn_conv_rows_fwd": [_c_vp, _c_i64, _c_i64, _c_vp, _c_vp, _c_i64, _c_i32, _c_i32, _c_i32, _c_i32, _c_i32, _c_vp, _c_vp,
                          _c_vp, _c_i64, _c_i32, _c_vp, _c_i64, _c_i32, _c_vp, _c_vp],
}

_lib = None

# Kernels launched by one call of each entry point (0: host-only query).  Used to
# count this library's launches, e.g. by the benchmark harness.
KERNELS_PER_CALL = {
    "wcn_hash_build": 2, "wcn_hash_search": 1, "wcn_unique_mark": 3, "wcn_unique_emit": 2, "wcn_kmap_search": 1, "wcn_kmap_search_static": 3,
    "wcn_kmap_scan": 2, "wcn_kmap_compact": 1, "wcn_nbr_from_maps": 1, "wcn_nbr_transpose": 1, "wcn_morton20": 1,
    "wcn_kmap_tile_order": 3, "wcn_conv_wgrad": 1, "wcn_kmap_tile_masks": 1, "wcn_row_reduce": 1, "wcn_kmap_search_self": 1, "wcn_kmap_search_dilated": 1, "wcn_kmap_count": 1,
    "wcn_gather_rows": 1, "wcn_scatter_add_rows": 1, "wcn_conv_pack_weight": 1, "wcn_conv_fwd": 1,
    "wcn_selftest_bounded_wait": 1, "wcn_brick_build": 3, "wcn_kmap_search_bricks": 1,
    "wcn_conv_rows_fwd": 1,
}
LAUNCH_COUNTS: Counter = Counter()


class _CountingLib:
    """Attribute access returns the C function wrapped so that calls are counted."""

    def __init__(self, handle):
        self._handle = handle
        self._wrapped = {}

    def __getattr__(self, name):
        fn = self._wrapped.get(name)
        if fn is None:
            raw = getattr(self._handle, name)
            n = KERNELS_PER_CALL.get(name, 0)
            if n:
                def fn(*args, _raw=raw, _name=name, _n=n):
                    LAUNCH_COUNTS[_name] += _n
                    return _raw(*args)
            else:
                fn = raw
            self._wrapped[name] = fn
        return fn


def launches_total() -> int:
    return sum(LAUNCH_COUNTS.values())


class NativeLibraryError(RuntimeError):
    pass


def lib():
    """The loaded library; raises NativeLibraryError when it is not built."""
    global _lib
    if _lib is None:
        if not os.path.isfile(LIB_PATH):
            raise NativeLibraryError(
                f"{LIB_PATH} is missing: build it with `python -m warpconvnet_b200.csrc.build` "
                "(nvcc, sm_100a). This package has no fallback path.")
        try:
            handle = ctypes.CDLL(LIB_PATH)
        except OSError as e:  # pragma: no cover
            raise NativeLibraryError(f"cannot load {LIB_PATH}: {e}") from e
        for name, argtypes in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.argtypes = argtypes
            fn.restype = ctypes.c_int
        handle.wcn_status_string.argtypes = [ctypes.c_int]
        handle.wcn_status_string.restype = ctypes.c_char_p
        handle.wcn_brick_usable_flag.argtypes = [ctypes.c_void_p]
        handle.wcn_brick_usable_flag.restype = ctypes.c_void_p
        _lib = _CountingLib(handle)
    return _lib


def status_string(status: int) -> str:
    return lib().wcn_status_string(int(status)).decode()


def check(status: int, what: str = "") -> None:
    if status != 0:
        raise RuntimeError(f"libwcn_b200 {what} failed: {status_string(status)} ({status})")


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream_ptr(device: torch.device) -> int:
    """Raw handle of torch's current stream on ``device`` (the launches go there)."""
    idx = device.index
    if idx is None:
        idx = torch.cuda.current_device()
    return torch._C._cuda_getCurrentRawStream(idx)


def small_to_device(t: torch.Tensor, device, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """A small host tensor (batch offsets, a few sizes) on ``device`` WITHOUT synchronising the
    stream: staged through pinned memory and copied asynchronously.  (A plain ``.to(device)`` of
    pageable memory waits for everything queued on the stream before it returns.)"""
    if t.device.type != "cpu":
        return t.to(device=device, dtype=dtype)
    if dtype is not None and t.dtype != dtype:
        t = t.to(dtype)
    return t.pin_memory().to(device, non_blocking=True)


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise TypeError(f"unsupported feature dtype {dtype}; expected float32, float16 or bfloat16")


def require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be on a CUDA device, got {t.device}")


_status_words = {}


def device_status(device: torch.device) -> torch.Tensor:
    """Per-device int32 status word shared by all kernels that can fail on the device."""
    device = torch.device(device)
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    if key not in _status_words:
        _status_words[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status_words[key]


def raise_for_status(code: int, device: torch.device) -> None:
    """Raise for a status-word value the caller has already brought to the host; the word is
    zeroed so that the next launches run again."""
    if code != 0:
        device_status(device).zero_()
        raise RuntimeError(f"libwcn_b200 kernel reported: {status_string(int(code))} ({int(code)})")


def check_device_status(device: torch.device) -> None:
    """Read the status word (synchronises) and raise if a kernel recorded a failure.

    Kernels report hash-table overflow, an expired bounded wait and out-of-range indices only
    through this word, and the tensor-core kernels do no work while it is set (convolution
    outputs are then filled with NaN).  The package reads it wherever it synchronises with the
    host anyway (sizing strided coordinates, compacting a kernel map); a caller that never reaches
    such a point should call this after the work it wants checked."""
    raise_for_status(int(device_status(device).item()), device)


def query_bytes(fn_name: str, *args) -> int:
    out = ctypes.c_int64(0)
    check(getattr(lib(), fn_name)(*args, ctypes.byref(out)), fn_name)
    return int(out.value)
