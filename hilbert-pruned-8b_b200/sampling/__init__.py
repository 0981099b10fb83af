from .sampler import Sampler, SamplingParams, option_scores, uniform_from

__all__ = ["Sampler", "SamplingParams", "option_scores", "uniform_from"]
