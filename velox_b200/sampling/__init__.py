from .params import SamplingParams
from .rng import uniform

__all__ = ["SamplingParams", "uniform"]
