from .options import SamplingOptions, SamplingOptionsBuilder
from .philox import uniform as philox_uniform
from .sampler import BatchSampler, RequestSampling
