from .sampler import Sampler, SamplingOptions

__all__ = ["Sampler", "SamplingOptions"]
