from .step import ModelRunner, StepEntry, StepError
