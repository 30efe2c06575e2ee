"""inferloop_b200: a small, whole inference engine for one B200 (sm_100a).

    from inferloop_b200 import Engine, SamplingParams
    engine = Engine("/path/to/model_folder", dtype="bfloat16")
    tokens = engine.generate([[1, 2, 3]], SamplingParams(temperature=0.0), max_new_tokens=16)
"""
__version__ = "0.1.0"

from .sampling.params import SamplingParams  # noqa: E402


def __getattr__(name):
    # The engine pulls in torch and the kernels; load it on first use.
    if name in ("Engine", "TokenOutput"):
        from .engine import engine as _e
        return getattr(_e, name)
    if name in ("ModelRunner", "StepEntry"):
        from . import engine as _pkg
        return getattr(_pkg, name)
    raise AttributeError(name)


__all__ = ["Engine", "SamplingParams", "ModelRunner", "StepEntry", "TokenOutput"]
