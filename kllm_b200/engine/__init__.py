from .engine import Engine, Options
from .scheduler import Request, Scheduler
from .step import StepEntry, StepError, StepRunner

__all__ = ["Engine", "Options", "Request", "Scheduler", "StepEntry", "StepError", "StepRunner"]
