from .params import SamplingParams
from .defaults import GenerationDefaults
from . import host

__all__ = ["SamplingParams", "host"]
