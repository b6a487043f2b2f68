"""The engine: the model with its step function, and the generation loop above it."""
from .batch import SeqStep, StepContext, pack_step
from .model import Model, StepError, parameter_table, resolve_dtype
from .decode import DecodeRunner
from .generate import Completion, Engine, generate, plan_batch
from .runner import ModelEngine, generate_with_model
from .diagnostics import Diagnostics

__all__ = ["SeqStep", "StepContext", "pack_step", "Model", "StepError", "parameter_table", "resolve_dtype",
           "DecodeRunner", "Completion", "Engine", "generate", "plan_batch", "ModelEngine", "generate_with_model",
           "Diagnostics"]
