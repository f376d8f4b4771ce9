"""The model, the step function, the scheduler and the Python entry point."""

from .batch import RowInput, StepBatch
from .model import DecoderModel, build_model
from .llm import (LLM, Completed, ServeResult, batched_greedy_decode, generate,
                  generate_with_logprobs, serve_continuous, serve_static_wave)
from .runner import DTYPES, ModelRunner, OutOfPages, load_model
from .scheduler import Request, Scheduler

__all__ = ["LLM", "Completed", "Request", "Scheduler", "ServeResult", "batched_greedy_decode",
           "generate",
           "generate_with_logprobs", "serve_continuous", "serve_static_wave", "DTYPES", "DecoderModel", "ModelRunner", "OutOfPages", "RowInput", "StepBatch",
           "build_model", "load_model"]
