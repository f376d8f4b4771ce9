"""The model, the step function, the scheduler and the Python entry point."""

from .batch import RowInput, StepBatch
from .model import DecoderModel, build_model
from .runner import DTYPES, ModelRunner, OutOfPages, load_model

__all__ = ["DTYPES", "DecoderModel", "ModelRunner", "OutOfPages", "RowInput", "StepBatch",
           "build_model", "load_model"]
