from .runner import ModelRunner, StepEntry
from .loading import LoadedModel, load_model
from .scheduler import Scheduler, SchedulerOutput, ScheduledSeq
from .sequence import Sequence, SequenceStatus
from .llm import LLM, LLMEngine, RequestOutput, EngineStats
from .trace import TraceReplayer, replay_stream

__all__ = ["ModelRunner", "StepEntry", "LoadedModel", "load_model", "Scheduler", "SchedulerOutput",
           "ScheduledSeq", "Sequence", "SequenceStatus", "LLM", "LLMEngine", "RequestOutput",
           "EngineStats", "TraceReplayer", "replay_stream"]
