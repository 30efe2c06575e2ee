from .params import SamplingParams
from . import host

__all__ = ["SamplingParams", "host"]
