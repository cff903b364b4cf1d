from .engine import GptEngine, engine_with_random_weights
from .model import Block, Model
from .scheduler import Request, Scheduled, Scheduler, SchedulerOptions
from .step import StepEntry, StepError, StepRunner

__all__ = ["Block", "GptEngine", "Model", "Request", "Scheduled", "Scheduler", "SchedulerOptions", "StepEntry",
           "StepError", "StepRunner", "engine_with_random_weights"]
