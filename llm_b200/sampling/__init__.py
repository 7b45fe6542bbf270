from .sampler import SampleHandle, Sampler, SamplingParams, uniform_for

__all__ = ["SampleHandle", "Sampler", "SamplingParams", "uniform_for"]
