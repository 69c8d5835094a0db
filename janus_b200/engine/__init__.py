from .model import DecoderModel, model_weight_specs
from .step import Engine, EngineOptions, StepContext, StepEntry, StepError
from .workspace import Workspace

__all__ = ["DecoderModel", "model_weight_specs", "Engine", "EngineOptions", "StepContext", "StepEntry",
           "StepError", "Workspace"]
