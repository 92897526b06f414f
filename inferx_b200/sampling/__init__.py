from .params import SamplingParams  # noqa: F401
from .sampler import Sampler  # noqa: F401
