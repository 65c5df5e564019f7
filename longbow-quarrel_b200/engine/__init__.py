from .engine import Engine
from .model import Model
from .step import StepError

__all__ = ["Engine", "Model", "StepError"]
