from .runner import ModelRunner, StepResult
from .llm import LLM, Generator, RequestOutput, GenerateOutput

__all__ = ["ModelRunner", "StepResult", "LLM", "Generator", "RequestOutput", "GenerateOutput"]
