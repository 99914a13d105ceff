from .step import StepEntry, StepError, StepRunner
