from .params import SamplingParams
from .sampler import Sampler, SplitMix64, pick_from_pool, pool_size
