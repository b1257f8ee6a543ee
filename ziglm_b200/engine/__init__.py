from .batch import BatchLayout, StepContext
from .engine import Engine, EngineOptions, StepError
from .generate import (GenerationOptions, GenerationResult, GenerationStats, plan_batch, run_generation)
from .model import Model, declare_parameters
from .workspace import Workspace

__all__ = ["BatchLayout", "StepContext", "Engine", "EngineOptions", "StepError", "GenerationOptions",
           "GenerationResult", "GenerationStats", "plan_batch", "run_generation", "Model", "declare_parameters",
           "Workspace"]
