"""Marker base class of modules that take and return geometries
(warpconvnet/nn/modules/base_module.py)."""
import torch.nn as nn


class BaseSpatialModule(nn.Module):
    @property
    def device(self):
        return next(self.parameters()).device
