from .sampler import GREEDY, Sampler, SamplingParams, SamplingState

__all__ = ["GREEDY", "Sampler", "SamplingParams", "SamplingState"]
