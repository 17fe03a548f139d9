from .batch import StepBatch, build_batch
from .generate import Completion, plan_batches, run_generation

__all__ = ["StepBatch", "build_batch", "Completion", "plan_batches", "run_generation",
           "Engine", "StepError", "LM", "tensor_needs_of"]


def __getattr__(name):
    # the device-facing classes load the kernel library; import them on demand
    if name in ("Engine", "StepError"):
        from . import step
        return getattr(step, name)
    if name in ("LM", "tensor_needs_of"):
        from . import lm
        return getattr(lm, name)
    raise AttributeError(name)
