from .batch import DEVICE_TOKEN, BatchBuilder, BatchCapacity, StepBatch, StepEntry
from .scheduler import Engine, EngineConfig, Request, RequestTooLarge, State

__all__ = ["DEVICE_TOKEN", "BatchBuilder", "BatchCapacity", "StepBatch", "StepEntry", "Engine", "EngineConfig", "Request",
           "RequestTooLarge", "State", "StepFunction"]


def __getattr__(name):
    if name == "StepFunction":
        from .step import StepFunction
        return StepFunction
    raise AttributeError(name)
