from .params import DEFAULT_MAX_TOKENS, GREEDY, InvalidParameter, SamplingParams
from .sampler import Sampler, pack_options, philox4x32_10, reference_sample, uniform

__all__ = ["DEFAULT_MAX_TOKENS", "GREEDY", "InvalidParameter", "SamplingParams", "Sampler", "pack_options", "philox4x32_10",
           "reference_sample", "uniform"]
