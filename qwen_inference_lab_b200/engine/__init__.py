from .step import StepEntry, StepError, StepRunner
from .scheduler import Request, Scheduler, Work
from .engine import Engine
