from .params import SamplerParams
from .rng import mix64, request_seed, uniform01

__all__ = ["SamplerParams", "mix64", "request_seed", "uniform01"]
