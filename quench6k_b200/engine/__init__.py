from .batch import StepContext, StepEntry
from .runner import ModelRunner
from .scheduler import Request, ScheduledStep, Scheduler, FINISH_CANCELLED, FINISH_LENGTH, FINISH_STOP
from .engine import Engine, RequestOutput
