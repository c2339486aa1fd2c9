"""The step function, the scheduler and the engine loop above them."""
from .scheduler import Scheduler

__all__ = ["ModelRunner", "StepContext", "StepEntry", "Scheduler", "LLMEngine", "RequestOutput"]


def __getattr__(name):
    # everything that needs torch and the kernels is loaded on demand, so the
    # scheduler and the cache bookkeeping can be used without a device
    if name in ("ModelRunner", "StepContext", "StepEntry"):
        from . import step
        return getattr(step, name)
    if name in ("LLMEngine", "RequestOutput"):
        from . import llm_engine
        return getattr(llm_engine, name)
    raise AttributeError(name)
