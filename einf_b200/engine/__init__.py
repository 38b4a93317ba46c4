"""The engine: step function, executors, serving loop."""
from ..cache.control import (
    BatchPlan,
    ExecutionResult,
    RequestResult,
    RequestSpec,
    ScheduledRequest,
    Scheduler,
)
from .batch import BatchError, StepInputBuilder
from .executor import FakeExecutor, GpuExecutor
from .runner import ModelRunner, StepError, StepOutput
from .server import Engine, LLMServer

__all__ = [
    "BatchError",
    "BatchPlan",
    "Engine",
    "ExecutionResult",
    "FakeExecutor",
    "GpuExecutor",
    "LLMServer",
    "ModelRunner",
    "RequestResult",
    "RequestSpec",
    "ScheduledRequest",
    "Scheduler",
    "StepError",
    "StepInputBuilder",
    "StepOutput",
]
