from .batch import StepContext, StepEntry
from .scheduler import Request, RequestRefused, Scheduler, SchedulerStats

__all__ = ["StepContext", "StepEntry", "Request", "RequestRefused", "Scheduler", "SchedulerStats", "Engine",
           "ModelRunner"]


def __getattr__(name):
    if name == "Engine":
        from .engine import Engine
        return Engine
    if name == "ModelRunner":
        from .step import ModelRunner
        return ModelRunner
    raise AttributeError(name)
