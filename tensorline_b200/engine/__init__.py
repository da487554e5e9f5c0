"""The engine: step function (`ModelRunner`), scheduler, and the `Engine` entry point."""
from .runner import ModelRunner, StepEntry, StepContext
from .scheduler import Scheduler, Request, RequestDoesNotFit
from .engine import Engine, Output

__all__ = ["ModelRunner", "StepEntry", "StepContext", "Scheduler", "Request", "RequestDoesNotFit", "Engine", "Output"]
