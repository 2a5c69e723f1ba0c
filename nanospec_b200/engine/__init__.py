from .step import ModelRunner, StepEntry

__all__ = ["ModelRunner", "StepEntry"]
