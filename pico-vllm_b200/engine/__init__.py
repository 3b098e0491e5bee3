from .batch import Batch, GroupBatch
from .runner import ModelRunner, StepItem
from .scheduler import Scheduler, Request, RequestStatus, Scheduled
from .core import load_model, model_from_tensors, make_cache, make_runner

__all__ = ["Batch", "GroupBatch", "ModelRunner", "StepItem", "load_model", "model_from_tensors",
           "make_cache", "make_runner", "Scheduler", "Request", "RequestStatus", "Scheduled"]
