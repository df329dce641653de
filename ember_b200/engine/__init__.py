"""Step function, scheduler, engine and trace replay."""
from .batch import BatchError, StepBatch, StepEntry, build_batch

__all__ = ["BatchError", "StepBatch", "StepEntry", "build_batch"]
