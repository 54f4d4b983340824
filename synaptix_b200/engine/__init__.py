from .generate import (GenerationOptions, GenerationResult, GenerationStats, plan_batches,
                       run_generation)
from .step import DecodeRun, Engine, Entry, StepError

__all__ = ["DecodeRun", "Engine", "Entry", "StepError", "GenerationOptions", "GenerationResult", "GenerationStats",
           "plan_batches", "run_generation"]
