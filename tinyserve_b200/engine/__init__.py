from .arena import Arena
from .engine import Engine, RequestTimes, StepRecord
from .llm import LLM
from .replay import Replayer
from .request import Request, Status
from .scheduler import Scheduler
from .step import ModelRunner, StepEntry

__all__ = ["Arena", "Engine", "RequestTimes", "StepRecord", "LLM", "Replayer", "Request", "Status",
           "Scheduler", "ModelRunner", "StepEntry"]
