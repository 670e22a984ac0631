from .step import ModelRunner, StepEntry, StepError
from .scheduler import RequestRejected, ScheduledItem, Scheduler, SeqState
from .llm import LLM, GenerationResult
