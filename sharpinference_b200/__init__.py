"""sharpinference_b200: a small, whole inference engine for one B200.

From a model folder (``config.json`` + ``model.safetensors``) to generated tokens: a typed
configuration and an architecture registry, weights by tensor name, layers put together from
parts, a paged cache manager, one step function, a scheduler, a sampler, and hand-written
sm_100a kernels beneath.  See ``Engine`` for the entry point.
"""
from .config import ConfigError, Llama4TextConfig
from .engine import Engine, EngineOptions, RequestOutput, StepEntry
from .registry import get_architecture, known_architectures, register_architecture
from .sampling import SamplingParams
from .weights import WeightError, build_random_model, load_model, write_random_model

__version__ = "0.1.0"

__all__ = ["ConfigError", "Llama4TextConfig", "Engine", "EngineOptions", "RequestOutput", "StepEntry",
           "get_architecture", "known_architectures", "register_architecture", "SamplingParams", "WeightError",
           "build_random_model", "load_model", "write_random_model"]
