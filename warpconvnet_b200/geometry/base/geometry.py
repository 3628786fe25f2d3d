"""``Geometry``: coordinates + features + free-form extra attributes.

Same surface as the reference base class (warpconvnet/geometry/base/geometry.py:37-347):
``replace`` shallow-copies the extra attributes (so the kernel-map cache object is
shared by every tensor derived from one input), ``feature_tensor`` follows the
autocast dtype, arithmetic acts on the features.
"""
from __future__ import annotations

from typing import Any, Dict, Optional, Union

import torch
from torch import Tensor

from ..coords.ops.batch_index import batch_indexed_coordinates
from ..features.cat import CatFeatures, to_batched_features
from .batched import Coords, Features


def _amp(tensor: Tensor) -> Tensor:
    # geometry.py:17-34: under autocast, features are seen in the autocast dtype
    if torch.is_autocast_enabled():
        amp_dtype = torch.get_autocast_gpu_dtype()
        if amp_dtype is not None:
            return tensor.to(dtype=amp_dtype)
    return tensor


class Geometry:
    batched_coordinates: Coords
    batched_features: Features
    _extra_attributes: Dict[str, Any]

    def __init__(self, batched_coordinates: Union[Coords, Tensor],
                 batched_features: Union[CatFeatures, Tensor], **kwargs):
        offsets = kwargs.pop("offsets", None)
        if isinstance(batched_coordinates, Tensor):
            assert offsets is not None, "offsets must be provided when batched_coordinates is a tensor"
            batched_coordinates = Coords(batched_coordinates, offsets)
        self.batched_coordinates = batched_coordinates
        self.batched_features = to_batched_features(batched_features, batched_coordinates.offsets,
                                                    device=kwargs.get("device", None))
        a, b = batched_coordinates.offsets, self.batched_features.offsets
        assert a is b or bool((a.long() == b.long()).all())
        if "_extra_attributes" in kwargs:
            attr = kwargs.pop("_extra_attributes")
            assert isinstance(attr, dict), f"_extra_attributes must be a dictionary, got {attr}"
            kwargs.update(attr)
        self._extra_attributes = kwargs

    def __getitem__(self, idx: int) -> "Geometry":
        coords = self.batched_coordinates[idx]
        feats = self.batched_features[idx]
        return self.__class__(batched_coordinates=coords, batched_features=feats,
                              offsets=torch.tensor([0, len(coords)]), **self._extra_attributes)

    def to(self, device=None, dtype: Optional[torch.dtype] = None) -> "Geometry":
        if device is None:
            device = self.device
        return self.__class__(batched_coordinates=self.batched_coordinates.to(device=device),
                              batched_features=self.batched_features.to(device=device, dtype=dtype),
                              **self._extra_attributes)

    # -- tensors
    @property
    def num_spatial_dims(self) -> int:
        return self.batched_coordinates.num_spatial_dims

    @property
    def coordinate_tensor(self) -> Tensor:
        return self.batched_coordinates.batched_tensor

    coordinates = coordinate_tensor

    @property
    def batch_indexed_coordinates(self) -> Tensor:
        return batch_indexed_coordinates(self.coordinate_tensor, self.offsets)

    @property
    def feature_tensor(self) -> Tensor:
        return _amp(self.batched_features.batched_tensor)

    features = feature_tensor

    @property
    def offsets(self) -> Tensor:
        return self.batched_features.offsets

    @property
    def device(self):
        return self.batched_features.device

    @property
    def num_channels(self) -> int:
        return self.batched_features.num_channels

    @property
    def batch_size(self) -> int:
        return len(self.offsets) - 1

    @property
    def dtype(self):
        return self.batched_features.dtype

    def __len__(self) -> int:
        return len(self.batched_coordinates)

    def numel(self):
        return self.offsets[-1] * self.num_channels

    @property
    def extra_attributes(self):
        return self._extra_attributes.copy()

    @property
    def cache(self):
        return self._extra_attributes.get("_cache")

    # -- functional updates
    def replace(self, batched_coordinates: Optional[Coords] = None,
                batched_features: Optional[Union[CatFeatures, Tensor]] = None, **kwargs):
        if "_extra_attributes" in kwargs:
            kwargs = {**kwargs.pop("_extra_attributes"), **kwargs}
        coords = batched_coordinates if batched_coordinates is not None else self.batched_coordinates
        feats = batched_features if batched_features is not None else self.batched_features
        if isinstance(feats, Tensor):
            feats = to_batched_features(feats, coords.offsets)
        return self.__class__(coords, feats, **{**self._extra_attributes, **kwargs})

    def _derive(self, features: Tensor, coords: Optional[Coords] = None) -> "Geometry":
        """Same kind of object with ``features`` (``[N, C]`` for the rows of ``coords``, default this
        object's coordinates) and the same extra attributes.  For results whose row count is already
        guaranteed by the kernel that made them; unlike ``replace`` it checks and converts nothing."""
        new = object.__new__(self.__class__)
        c = coords if coords is not None else self.batched_coordinates
        f = object.__new__(CatFeatures)
        f.batched_tensor = features
        f.offsets = c.offsets
        new.batched_coordinates = c
        new.batched_features = f
        new._extra_attributes = dict(self._extra_attributes)
        return new

    def _apply_feature_transform(self, fn):
        return self.replace(batched_features=fn(self.feature_tensor))

    def half(self):
        return self._apply_feature_transform(lambda x: x.half())

    def float(self):
        return self._apply_feature_transform(lambda x: x.float())

    def double(self):
        return self._apply_feature_transform(lambda x: x.double())

    def equal_shape(self, value: object) -> bool:
        if isinstance(value, Tensor):
            return tuple(value.shape) == tuple(self.feature_tensor.shape)
        return (self.batched_coordinates.equal_shape(value.batched_coordinates)
                and self.batched_features.equal_shape(value.batched_features))

    def binary_op(self, value: object, op: str) -> "Geometry":
        if isinstance(value, Geometry):
            assert self.equal_shape(value), f"Shapes do not match. {self} != {value}"
            return self._apply_feature_transform(lambda x: getattr(x, op)(value.feature_tensor))
        if isinstance(value, (int, float)) or (torch.is_tensor(value) and value.numel() == 1):
            return self._apply_feature_transform(lambda x: getattr(x, op)(value))
        if isinstance(value, Tensor):
            assert self.equal_shape(value)
            return self._apply_feature_transform(lambda x: getattr(x, op)(value))
        raise NotImplementedError

    def __add__(self, value):
        return self.binary_op(value, "__add__")

    def __sub__(self, value):
        return self.binary_op(value, "__sub__")

    def __mul__(self, value):
        return self.binary_op(value, "__mul__")

    def __truediv__(self, value):
        return self.binary_op(value, "__truediv__")

    def sort(self):
        raise NotImplementedError

    def __str__(self) -> str:
        return (f"{self.__class__.__name__}(feature_shape={tuple(self.feature_tensor.shape)}, "
                f"coords_shape={tuple(self.batched_coordinates.shape)})")

    def __repr__(self) -> str:
        out = (f"{self.__class__.__name__}(offsets={self.offsets.tolist()}, "
               f"feature_shape={tuple(self.feature_tensor.shape)}, "
               f"coords_shape={tuple(self.batched_coordinates.shape)}, device={self.device}, "
               f"dtype={self.feature_tensor.dtype}")
        extras = {k: v for k, v in self._extra_attributes.items() if v is not None and not k.startswith("_")}
        if extras:
            out += ", " + ", ".join(f"{k}={v}" for k, v in extras.items())
        return out + ")"
