from .batch import GroupBatch, StepBatch, build_step_batch
from .engine import Engine, StepEntry, StepError
from .model import DecoderModel, parameter_requests
