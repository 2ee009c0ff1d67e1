"""Step function, scheduler, entry point and trace replay."""
from .batch import Portion
from .engine import Engine
from .runner import ModelRunner
from .scheduler import Request, Scheduler, StepPlan

__all__ = ["Portion", "Engine", "ModelRunner", "Request", "Scheduler", "StepPlan"]
