from .batch import AttentionMeta, SequenceInput, StepBatch, build_step_batch
from .engine import Engine, RequestOutput
from .request import Request, RequestState
from .runner import ModelRunner
from .scheduler import Scheduled, Scheduler
