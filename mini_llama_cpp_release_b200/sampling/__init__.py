from .rng import uniform_of  # noqa: F401
from .sampler import DeviceSampler, HostSampler, SamplingParams  # noqa: F401
