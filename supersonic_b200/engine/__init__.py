"""The step function, the generation loop above it, and trace replay."""
from .batch import StepBatch, StepEntry, batch_over, pack_entries, pack_step, plan_chunks
from .model import Model, StepContext, parse_dtype

__all__ = ["StepBatch", "StepEntry", "batch_over", "pack_entries", "pack_step", "plan_chunks", "Model", "StepContext", "parse_dtype"]
