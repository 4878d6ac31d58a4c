from .runner import ModelRunner, StepResult

__all__ = ["ModelRunner", "StepResult"]
