from .batch import BatchBuilder, StepBatch, StepEntry

__all__ = ["BatchBuilder", "StepBatch", "StepEntry"]
