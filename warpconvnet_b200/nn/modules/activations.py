"""Activations on geometry features (warpconvnet/nn/modules/activations.py:36-53)."""
import torch.nn as nn

from ...geometry.base.geometry import Geometry
from ..functional.transforms import apply_feature_transform
from .base_module import BaseSpatialModule


class ReLU(BaseSpatialModule):
    def __init__(self, inplace: bool = False):
        super().__init__()
        self.relu = nn.ReLU(inplace=inplace)

    def __repr__(self):
        return f"{self.__class__.__name__}(inplace={self.relu.inplace})"

    def forward(self, input: Geometry):
        return apply_feature_transform(input, self.relu)
