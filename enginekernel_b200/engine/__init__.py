"""Model assembly, the step function, decoding on the device, the generation loop."""
from .engine import Engine
from .generate import GenerationError, GenerationLoop
from .loading import load_model, random_model
from .model import DecoderModel, expected_tensors
from .runner import ModelRunner, StepEntry, StepError

__all__ = ["Engine", "GenerationError", "GenerationLoop", "load_model", "random_model",
           "DecoderModel", "expected_tensors", "ModelRunner", "StepEntry", "StepError"]
