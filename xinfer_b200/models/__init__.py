"""Models: the generic decoder that builds any registered architecture's plan."""
from .decoder import DecoderModel, model_weight_specs

__all__ = ["DecoderModel", "model_weight_specs"]
