from .params import SamplingParams, uniform_from

__all__ = ["SamplingParams", "uniform_from", "Sampler"]


def __getattr__(name):
    if name == "Sampler":
        from .sampler import Sampler
        return Sampler
    raise AttributeError(name)
