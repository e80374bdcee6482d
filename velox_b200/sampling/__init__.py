from .params import SamplingParams
from .rng import uniform

__all__ = ["SamplingParams", "uniform", "Sampler"]


def __getattr__(name):
    if name == "Sampler":  # needs the kernels; everything else here does not
        from .sampler import Sampler
        return Sampler
    raise AttributeError(name)
