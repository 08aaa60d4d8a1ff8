from .step import StepEntry, StepRunner, DeviceFault
from .scheduler import Scheduler, SchedulerError, StepPlan, PlannedEntry
from .engine import Engine, RequestOutput

__all__ = ["StepEntry", "StepRunner", "DeviceFault", "Scheduler", "SchedulerError", "StepPlan",
           "PlannedEntry", "Engine", "RequestOutput"]
