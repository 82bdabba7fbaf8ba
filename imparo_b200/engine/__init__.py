from .engine import Engine
from .scheduler import PlanEntry, Scheduler
from .step import StepBatch, StepFunction, StepItem

__all__ = ["Engine", "Scheduler", "PlanEntry", "StepFunction", "StepItem", "StepBatch"]
