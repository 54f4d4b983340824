from .generate import (GenerationOptions, GenerationResult, GenerationStats, plan_batches,
                       run_generation)
from .step import Engine, Entry, StepError

__all__ = ["Engine", "Entry", "StepError", "GenerationOptions", "GenerationResult", "GenerationStats",
           "plan_batches", "run_generation"]
