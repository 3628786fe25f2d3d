"""Feature-wise helpers on geometries (warpconvnet/nn/functional/transforms.py:40-85)."""
from typing import Sequence

import torch

from ...geometry.base.geometry import Geometry


def apply_feature_transform(input: Geometry, transform) -> Geometry:
    assert isinstance(input, Geometry), f"Expected Geometry, got {type(input)}"
    return input.replace(batched_features=transform(input.feature_tensor))


def cat(*inputs: Geometry, dim: int = -1):
    """Concatenate the features of geometries that share coordinates (skip connections)."""
    if len(inputs) == 1 and isinstance(inputs[0], Sequence):
        inputs = inputs[0]
    assert all(isinstance(i, Geometry) for i in inputs), f"Expected all inputs to be Geometry, got {type(inputs)}"
    assert all(torch.equal(i.offsets.long(), inputs[0].offsets.long()) for i in inputs), \
        "All inputs must have the same offsets"
    return inputs[0].replace(batched_features=torch.cat([i.feature_tensor for i in inputs], dim=dim))
