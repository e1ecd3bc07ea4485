from .step import StepEntry, StepContext, ModelRunner
from .scheduler import Scheduler, Request, ScheduledBatch, ScheduledEntry
from .core import Engine
from .llm import LLM, RequestOutput, CompletionOutput
