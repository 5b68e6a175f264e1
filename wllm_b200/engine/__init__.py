from .build import build_model, build_runner
from .model import ComposedModel
from .runner import ModelRunner, StepContext, StepEntry

__all__ = ["build_model", "build_runner", "ComposedModel", "ModelRunner", "StepContext", "StepEntry"]
