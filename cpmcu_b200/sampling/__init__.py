from .sampler import SamplingParams

__all__ = ["SamplingParams"]
