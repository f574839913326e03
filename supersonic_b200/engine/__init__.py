"""The step function, the generation loop above it, and trace replay."""
from .batch import StepBatch, StepEntry, pack_step
from .model import Model, StepContext, parse_dtype

__all__ = ["StepBatch", "StepEntry", "pack_step", "Model", "StepContext", "parse_dtype"]
