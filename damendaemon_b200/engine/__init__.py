from .engine import Engine, StepEntry, StepError

__all__ = ["Engine", "StepEntry", "StepError"]
