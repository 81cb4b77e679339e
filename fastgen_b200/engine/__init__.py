from .model import Model, model_weight_specs
from .step import Engine, StepContext, StepEntry

__all__ = ["Engine", "Model", "StepContext", "StepEntry", "model_weight_specs"]
