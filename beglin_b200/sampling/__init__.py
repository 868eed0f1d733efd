from .sampler import Sampler, SamplingParams, request_key, uniform

__all__ = ["Sampler", "SamplingParams", "request_key", "uniform"]
