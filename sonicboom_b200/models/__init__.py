"""Whole models: the generic decoder over a ModelSpec, and loading one from a folder."""
from .decoder import DecoderModel, tensor_requests
from .loading import load_model, random_model

__all__ = ["DecoderModel", "tensor_requests", "load_model", "random_model"]
