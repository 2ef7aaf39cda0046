from .engine import Engine, EngineConfig
from .llm import LLM
from .loading import load_model, parse_dtype
from .scheduler import (AddResult, Batch, FinishReason, ReqState, Request, Scheduler, SchedulerError, SchedulerStats,
                        StepResult, WorkItem, host_only_cache)
from .step import EngineError, ModelRunner, StepItem

__all__ = [
    "AddResult", "Batch", "Engine", "EngineConfig", "EngineError", "FinishReason", "LLM", "ModelRunner", "ReqState",
    "Request", "Scheduler", "SchedulerError", "SchedulerStats", "StepItem", "StepResult", "WorkItem",
    "host_only_cache", "load_model", "parse_dtype",
]
