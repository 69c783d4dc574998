from .model import Model, parse_dtype
from .step import ModelRunner, StepEntry, StepError

__all__ = ["Model", "ModelRunner", "StepEntry", "StepError", "parse_dtype"]
