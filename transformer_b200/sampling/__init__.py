from .args import SampleArgs, SampleArgsError, uniform
from .sampler import Sampler
