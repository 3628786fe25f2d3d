"""``CatFeatures``: features of a batch stored as one ``[N, C]`` tensor
(warpconvnet/geometry/features/cat.py:11-33)."""
from ..base.batched import Features


class CatFeatures(Features):
    def check(self):
        super().check()
        assert self.batched_tensor.ndim == 2, "Batched tensor must be 2D"

    @property
    def is_cat(self) -> bool:
        return True

    def equal_shape(self, value: object) -> bool:
        if not isinstance(value, CatFeatures):
            return False
        return (bool((self.offsets.long() == value.offsets.long()).all()) and self.numel() == value.numel()
                and self.num_channels == value.num_channels)


def to_batched_features(features, offsets, device=None):
    """Wrap a tensor (or pass through a Features object) as CatFeatures
    (warpconvnet/geometry/features/ops/convert.py: ``to_batched_features``)."""
    from torch import Tensor
    if isinstance(features, Tensor):
        assert features.ndim == 2, "only concatenated [N, C] features are supported"
        return CatFeatures(features, offsets, device=device)
    assert isinstance(features, CatFeatures), f"unsupported features type {type(features)}"
    if device is not None:
        features = features.to(device)
    return features
