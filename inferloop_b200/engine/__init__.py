from .batch import StepContext, StepEntry
from .runner import ModelRunner, parse_dtype, prepare_step

__all__ = ["StepContext", "StepEntry", "ModelRunner", "parse_dtype", "prepare_step"]
