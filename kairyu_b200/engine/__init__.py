from kairyu_b200.engine.engine import Engine, FinishedRequest, build_model, load_model, random_model
from kairyu_b200.engine.runner import ModelRunner, StepEntry, StepError
from kairyu_b200.engine.scheduler import EngineRequest, ScheduledChunk, Scheduler, SchedulerOutput

__all__ = [
    "Engine", "EngineRequest", "FinishedRequest", "ModelRunner", "ScheduledChunk", "Scheduler", "SchedulerOutput",
    "StepEntry", "StepError", "build_model", "load_model", "random_model",
]
