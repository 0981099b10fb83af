from .batch import StepBatch, StepEntry, build_step
from .model import DecoderModel, weight_table
from .workspace import Workspace

__all__ = ["StepBatch", "StepEntry", "build_step", "DecoderModel", "weight_table", "Workspace"]
