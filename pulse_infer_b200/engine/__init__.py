from .builder import build_model, build_runner
from .context import CacheView, Segment, StepContext
from .step import ModelRunner, StepError

__all__ = ["build_model", "build_runner", "CacheView", "Segment", "StepContext", "ModelRunner", "StepError"]
