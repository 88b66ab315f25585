"""Weights: safetensors by tensor name, and the random-weights mode."""
from .loading import build_random_model, declared_tensors, load_model, parse_dtype, write_random_model
from .source import DeclaringWeights, FileWeights, RandomWeights, TensorDecl, WeightError, WeightSource

__all__ = ["build_random_model", "declared_tensors", "load_model", "parse_dtype", "write_random_model",
           "DeclaringWeights", "FileWeights", "RandomWeights", "TensorDecl", "WeightError", "WeightSource"]
