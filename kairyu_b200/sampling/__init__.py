from kairyu_b200.sampling.params import SamplingParams
from kairyu_b200.sampling.rng import mix_seed, stable_request_seed
from kairyu_b200.sampling.sampler import Sampler, SamplingRow

__all__ = ["Sampler", "SamplingParams", "SamplingRow", "mix_seed", "stable_request_seed"]
