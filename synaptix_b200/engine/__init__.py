from .step import Engine, Entry, StepError

__all__ = ["Engine", "Entry", "StepError"]
