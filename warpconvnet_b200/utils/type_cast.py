"""dtype ranking used when features and weights differ
(warpconvnet/utils/type_cast.py:10-25): bf16 < fp16 < fp32 < fp64."""
from typing import Optional

import torch

TYPE_ORDER = [torch.bfloat16, torch.float16, torch.float32, torch.float64]


def _min_dtype(*dtypes):
    assert all(d in TYPE_ORDER for d in dtypes), f"Invalid dtype: {dtypes}"
    return TYPE_ORDER[min(TYPE_ORDER.index(d) for d in dtypes)]


def _max_dtype(*dtypes):
    assert all(d in TYPE_ORDER for d in dtypes), f"Invalid dtype: {dtypes}"
    return TYPE_ORDER[max(TYPE_ORDER.index(d) for d in dtypes)]


def _maybe_cast(tensor: torch.Tensor, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    return tensor if dtype is None else tensor.to(dtype=dtype)
