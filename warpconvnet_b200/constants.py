"""Environment-variable configuration of the sparse-convolution algorithms.

Same variables, values and list syntax as the reference
(warpconvnet/constants.py:95-117): ``WARPCONVNET_FWD_ALGO_MODE`` and
``WARPCONVNET_BWD_ALGO_MODE`` take ``explicit_gemm``, ``implicit_gemm``,
``cutlass_implicit_gemm``, ``auto`` or a bracketed list such as
``[implicit_gemm,cutlass_implicit_gemm]``; the default is ``auto``.
"""
import os
from typing import List, Union

VALID_ALGOS = ["explicit_gemm", "implicit_gemm", "cutlass_implicit_gemm", "auto"]


def _get_env_string_list(name: str, default: str, valid: List[str]) -> Union[str, List[str]]:
    raw = os.environ.get(name)
    if raw is None:
        return default
    raw = raw.strip()
    if raw.startswith("[") and raw.endswith("]"):
        items = [x.strip().strip("'\"").lower() for x in raw[1:-1].split(",") if x.strip()]
        for it in items:
            if it not in valid:
                raise ValueError(f"{name} has invalid value {it!r}; valid: {valid}")
        return items
    value = raw.lower()
    if value not in valid:
        raise ValueError(f"{name} has invalid value {raw!r}; valid: {valid}")
    return value


def _get_env_bool(name: str, default: bool) -> bool:
    raw = os.environ.get(name)
    if raw is None:
        return default
    return raw.strip().lower() in ("1", "true", "yes", "on")


WARPCONVNET_SKIP_SYMMETRIC_KERNEL_MAP = _get_env_bool("WARPCONVNET_SKIP_SYMMETRIC_KERNEL_MAP", False)
WARPCONVNET_FWD_ALGO_MODE = _get_env_string_list("WARPCONVNET_FWD_ALGO_MODE", "auto", VALID_ALGOS)
WARPCONVNET_BWD_ALGO_MODE = _get_env_string_list("WARPCONVNET_BWD_ALGO_MODE", "auto", VALID_ALGOS)
