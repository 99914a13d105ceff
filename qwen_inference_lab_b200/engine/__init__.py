from .step import StepEntry, StepError, StepRunner
from .scheduler import Scheduler, Sequence, Turn
from .engine import Engine
