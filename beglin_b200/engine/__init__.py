from .batch import Entry, StepBatch
from .scheduler import Request, Scheduler, StepPlan

__all__ = ["Entry", "StepBatch", "Request", "Scheduler", "StepPlan", "Engine"]


def __getattr__(name):
    if name == "Engine":
        from .engine import Engine
        return Engine
    raise AttributeError(name)
