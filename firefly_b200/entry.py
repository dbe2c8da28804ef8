"""Public Python entry point (re-exported at package level)."""
from .engine.engine import LLM, Engine, EngineOptions, ResultQueue, StepOutput
from .sampling.params import SamplingParams

__all__ = ["LLM", "Engine", "EngineOptions", "ResultQueue", "StepOutput", "SamplingParams"]
