from .generate import (GenerationOptions, GenerationResult, GenerationStats, plan_batches,
                       run_generation)
from .step import DecodeRow, DecodeSession, Engine, Entry, StepError

__all__ = ["DecodeRow", "DecodeSession", "Engine", "Entry", "StepError", "GenerationOptions", "GenerationResult",
           "GenerationStats", "plan_batches", "run_generation"]
