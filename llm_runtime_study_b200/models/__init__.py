from . import mabedra, qwen3, ropulix, sorulix, tafisun  # registers the architectures
from .description import LayerDescription, ModelDescription, tensor_schema
from .loading import load_model_dir, random_model
from .model import DecoderModel

__all__ = [
    "DecoderModel", "LayerDescription", "ModelDescription", "load_model_dir", "random_model", "tensor_schema",
]
