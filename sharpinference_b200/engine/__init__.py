"""The engine: step function, scheduler and the Python entry point."""
from .engine import Engine, EngineOptions, RequestOutput
from .scheduler import PlannedEntry, Request, Scheduler, StepPlan
from .step import StepEntry, StepError, StepRunner

__all__ = ["Engine", "EngineOptions", "RequestOutput", "PlannedEntry", "Request", "Scheduler", "StepPlan",
           "StepEntry", "StepError", "StepRunner"]
