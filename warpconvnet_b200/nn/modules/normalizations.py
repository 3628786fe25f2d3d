"""BatchNorm over geometry features (warpconvnet/nn/modules/normalizations.py:49-63)."""
import torch.nn as nn

from ...geometry.base.geometry import Geometry
from ..functional.transforms import apply_feature_transform
from .base_module import BaseSpatialModule


class BatchNorm(BaseSpatialModule):
    def __init__(self, num_features: int, eps: float = 1e-5, momentum: float = 0.1):
        super().__init__()
        self.norm = nn.BatchNorm1d(num_features, eps=eps, momentum=momentum)

    def __repr__(self):
        return f"{self.__class__.__name__}({self.norm})"

    def forward(self, input: Geometry):
        return apply_feature_transform(input, self.norm)
