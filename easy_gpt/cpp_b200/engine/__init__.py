from .model import Block, Model
from .step import StepEntry, StepError, StepRunner

__all__ = ["Block", "Model", "StepEntry", "StepError", "StepRunner"]
