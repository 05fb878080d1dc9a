from .scheduler import Planned, Request, Scheduler, SchedulerConfig
from .step import ModelRunner, StepEntry, StepError
