"""Engine: packed batches, the step function, the scheduler and the entry point."""
from .batch import BatchBuilder, StepBatch, StepEntry
from .runner import ModelRunner
from .scheduler import Request, Scheduled, Scheduler, SchedulerOutput

__all__ = ["BatchBuilder", "StepBatch", "StepEntry", "ModelRunner", "Request", "Scheduled",
           "Scheduler", "SchedulerOutput", "Engine"]


def __getattr__(name):
    if name == "Engine":
        from .engine import Engine
        return Engine
    raise AttributeError(name)
