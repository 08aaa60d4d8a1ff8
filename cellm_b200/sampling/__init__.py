from .params import SamplingParams
from .rng import XorShift64, session_seed
from .sampler import RequestSampler, sample_rows

__all__ = ["SamplingParams", "XorShift64", "session_seed", "RequestSampler", "sample_rows"]
