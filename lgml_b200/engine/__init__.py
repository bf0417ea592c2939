from .batch import CacheView, StepBatch
from .runner import ModelRunner, StepError
from .runtime import DeviceFault, Runtime

__all__ = ["CacheView", "StepBatch", "ModelRunner", "StepError", "DeviceFault", "Runtime"]
