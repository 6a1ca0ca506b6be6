from .params import SampleParams
from .sampler import Sampler, uniform_draw

__all__ = ["SampleParams", "Sampler", "uniform_draw"]
