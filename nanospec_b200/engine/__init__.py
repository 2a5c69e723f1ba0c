from .engine import Engine
from .scheduler import Request, RequestTooLarge, SamplingParams, Scheduled, Scheduler, TokenInfo
from .step import ModelRunner, StepEntry

__all__ = ["Engine", "ModelRunner", "Request", "RequestTooLarge", "SamplingParams", "Scheduled", "Scheduler",
           "StepEntry", "TokenInfo"]
