from .params import SamplerParams
from .sampler import DeviceSampler, SequenceSamplerState

__all__ = ["SamplerParams", "DeviceSampler", "SequenceSamplerState"]
