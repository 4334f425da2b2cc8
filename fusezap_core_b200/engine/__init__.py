from .model import DecoderModel, load_model, declared_tensors
from .step import Portion, Segment, StepMeta, StepRunner, StepContext, Workspace

__all__ = ["DecoderModel", "load_model", "declared_tensors", "Portion", "Segment", "StepMeta", "StepRunner",
           "StepContext", "Workspace"]
