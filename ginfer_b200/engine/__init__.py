from .runner import ModelRunner, StepEntry
from .request import Request, RequestState
from .scheduler import Scheduled, Scheduler
