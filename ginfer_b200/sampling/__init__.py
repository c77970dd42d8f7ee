from .params import SamplingParams
from .sampler import Sampler, uniform
