"""Concatenated ("cat") batches: one ``[N, C]`` tensor plus CPU ``offsets [B+1]``.

API of the reference's ``BatchedTensor`` / ``Coords`` / ``Features``
(warpconvnet/geometry/base/batched.py:14-263, base/coords.py, base/features.py),
reduced to what the sparse-convolution path touches.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Union

import torch
from torch import Tensor


def list_to_cat_tensor(tensors: Sequence[Tensor]):
    """Concatenate a list of ``[N_i, C]`` tensors; returns (tensor, int32 offsets, batch size)
    (warpconvnet/geometry/utils/list_to_batch.py:11-28)."""
    counts = torch.tensor([0] + [len(t) for t in tensors])
    offsets = counts.cumsum(dim=0).int()
    return torch.cat(list(tensors), dim=0), offsets, len(tensors)


def _as_cpu_offsets(offsets) -> Tensor:
    if isinstance(offsets, Tensor):
        if offsets.device.type == "cpu" and not offsets.requires_grad and offsets.dtype in (torch.int32, torch.int64):
            return offsets
        offsets = offsets.detach().cpu()
    elif isinstance(offsets, (list, tuple)):
        offsets = torch.tensor(list(offsets), dtype=torch.int64)
    else:
        raise ValueError(f"Invalid offsets type {type(offsets)}")
    if offsets.dtype not in (torch.int32, torch.int64):
        offsets = offsets.long()
    return offsets


class BatchedTensor:
    batched_tensor: Tensor
    offsets: Tensor  # CPU int32/int64 [B+1]

    def __init__(self, batched_tensor: Union[List[Tensor], Tensor], offsets=None,
                 device: Optional[Union[str, torch.device]] = None):
        if isinstance(batched_tensor, (list, tuple)):
            assert offsets is None, "If batched_tensors is a list, offsets must be None."
            batched_tensor, offsets, _ = list_to_cat_tensor(batched_tensor)
        else:
            assert isinstance(batched_tensor, Tensor), "Batched tensor must be a tensor or a list"
            if offsets is None:
                offsets = [0, batched_tensor.shape[0]]
        self.offsets = _as_cpu_offsets(offsets)
        if device is not None:
            batched_tensor = batched_tensor.to(device)
        self.batched_tensor = batched_tensor
        self.check()

    def check(self):
        assert self.offsets.device.type == "cpu" and self.offsets.dtype in (torch.int32, torch.int64), \
            f"Offsets must be a cpu IntTensor or cpu LongTensor, got {self.offsets}"
        assert not self.offsets.requires_grad, "Offsets must not require grad"
        assert isinstance(self.batched_tensor, Tensor)
        assert self.batched_tensor.shape[0] == int(self.offsets[-1]), \
            f"Offsets {self.offsets} does not match tensors {self.batched_tensor.shape}"

    # -- container protocol
    @property
    def batch_size(self) -> int:
        return len(self.offsets) - 1

    def __len__(self) -> int:
        return self.batched_tensor.shape[0]

    def __getitem__(self, idx: int) -> Tensor:
        return self.batched_tensor[int(self.offsets[idx]):int(self.offsets[idx + 1])]

    def numel(self):
        return self.batched_tensor.numel()

    @property
    def device(self):
        return self.batched_tensor.device

    @property
    def shape(self):
        return self.batched_tensor.shape

    @property
    def dtype(self):
        return self.batched_tensor.dtype

    def to(self, device=None, dtype: Optional[torch.dtype] = None):
        if device is None:
            device = self.device
        return self.__class__(self.batched_tensor.to(device=device, dtype=dtype), self.offsets)

    def half(self):
        return self.__class__(self.batched_tensor.half(), self.offsets)

    def float(self):
        return self.__class__(self.batched_tensor.float(), self.offsets)

    def double(self):
        return self.__class__(self.batched_tensor.double(), self.offsets)

    def equal_shape(self, value: object) -> bool:
        return (isinstance(value, BatchedTensor) and bool((self.offsets.long() == value.offsets.long()).all())
                and self.batched_tensor.shape == value.batched_tensor.shape)

    def to_nested(self):
        return torch.nested.nested_tensor([self[i] for i in range(self.batch_size)])

    def __repr__(self) -> str:
        return (f"{self.__class__.__name__}(offsets={self.offsets.tolist()}, shape={tuple(self.shape)}, "
                f"device={self.device}, dtype={self.dtype})")


def _operator(name: str):
    def apply(self: BatchedTensor, other):
        """Element-wise on the stored tensor; ``other`` is a scalar, a tensor that broadcasts against
        it, or another batch with the same offsets and shape (batched.py:183-229 of the reference)."""
        if isinstance(other, BatchedTensor):
            assert self.equal_shape(other), f"shapes do not match: {self} vs {other}"
            other = other.batched_tensor
        return self.__class__(getattr(self.batched_tensor, name)(other), self.offsets)
    apply.__name__ = name
    return apply


for _name in ("__add__", "__sub__", "__mul__", "__truediv__", "__floordiv__", "__mod__", "__pow__"):
    setattr(BatchedTensor, _name, _operator(_name))


class Coords(BatchedTensor):
    def check(self):
        BatchedTensor.check(self)
        assert self.batched_tensor.ndim == 2, "Coordinates must be [N, D]"

    @property
    def num_spatial_dims(self) -> int:
        return self.batched_tensor.shape[1]


class Features(BatchedTensor):
    @property
    def num_channels(self) -> int:
        return self.batched_tensor.shape[-1]

    @property
    def is_cat(self) -> bool:
        return False

    @property
    def is_pad(self) -> bool:
        return False
