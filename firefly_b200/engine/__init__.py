from .context import StepContext, Workspace
from .loading import load_model, parse_dtype, random_model
from .runner import ModelRunner, StepEntry, StepError

__all__ = ["StepContext", "Workspace", "load_model", "parse_dtype", "random_model", "ModelRunner",
           "StepEntry", "StepError"]
