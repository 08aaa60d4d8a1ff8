from .step import StepEntry, StepRunner, DeviceFault

__all__ = ["StepEntry", "StepRunner", "DeviceFault"]
