from .engine import (Engine, EngineConfig, GenerationResult, IterationResult, load_model,
                     parse_dtype, random_model, write_random_model)
from .metrics import DurationStatistics, SchedulerMetrics, observe
from .scheduler import (FifoScheduler, IterationBatch, Request, RequestState, ScheduledWork,
                        SchedulerConfig, StopReason, WorkCompletion, WorkKind)
from .step import StepEntry, StepError, StepFunction

__all__ = [
    "DurationStatistics", "Engine", "EngineConfig", "FifoScheduler", "GenerationResult", "IterationBatch",
    "IterationResult", "Request", "RequestState", "ScheduledWork", "SchedulerConfig",
    "SchedulerMetrics",
    "StepEntry", "StepError", "StepFunction", "StopReason", "WorkCompletion", "WorkKind",
    "load_model", "parse_dtype", "random_model", "observe",
    "write_random_model",
]
