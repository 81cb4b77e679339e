from .model import Model, model_weight_specs
from .step import Engine, StepContext, StepEntry

__all__ = ["Engine", "Model", "StepContext", "StepEntry", "model_weight_specs"]
from .generate import Fastgen, GenArgs, HfLoader, Packet  # noqa: E402
from .scheduler import Request, Scheduler  # noqa: E402

__all__ += ["Fastgen", "GenArgs", "HfLoader", "Packet", "Request", "Scheduler"]
