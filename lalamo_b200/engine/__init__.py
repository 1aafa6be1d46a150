"""The engine: step function, scheduler, generation, trace replay."""

from .engine import Engine, EngineConfig, NoDeviceError
from .executor import Executor, StepEntry, StepError

__all__ = ["Engine", "EngineConfig", "Executor", "NoDeviceError", "StepEntry", "StepError"]
