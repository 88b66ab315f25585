"""From a model folder (or a configuration and a seed) to a built model.

``load_model``: read config.json, pick the architecture from the registry, check every tensor
the architecture needs against the safetensors header (one error for all problems), then build.
``write_random_model``: the random-weights mode; it writes a model folder from a configuration
and a seed, which ``load_model`` reads like any other.
``build_random_model``: the same draws' distribution made directly on the device, without a file.
"""
from __future__ import annotations

import json
import os
from typing import List, Optional, Union

import torch

from ..config.base import read_config_json
from ..registry import Architecture, get_architecture, resolve
from . import safetensors_io
from .source import DeclaringWeights, FileWeights, RandomWeights, TensorDecl

_DTYPE_ALIASES = {
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16, torch.bfloat16: torch.bfloat16,
    "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32, torch.float32: torch.float32,
}


def parse_dtype(dtype) -> torch.dtype:
    try:
        return _DTYPE_ALIASES[dtype]
    except (KeyError, TypeError):
        raise ValueError(f"dtype must be 'bfloat16' or 'float32', found {dtype!r}") from None


def declared_tensors(arch: Architecture, config, compute_dtype: torch.dtype = torch.bfloat16,
                     stored_names=None) -> List[TensorDecl]:
    """Every tensor a model folder of this configuration must hold, in file order.  ``stored_names``: the
    names a folder does hold, for architectures that accept two layouts of the same weights (the declaration
    then asks for the layout that is there)."""
    decl = DeclaringWeights(compute_dtype, stored_names=stored_names, prefixes=("", "language_model."))
    arch.build(config, decl)
    return decl.decls


def load_model(model_dir: str, dtype="bfloat16", device="cuda:0"):
    """Build the model that ``model_dir/config.json`` names from ``model_dir/model.safetensors``."""
    compute = parse_dtype(dtype)
    obj = read_config_json(model_dir)
    arch, config = resolve(obj, os.path.join(model_dir, "config.json"))
    source = FileWeights(model_dir, compute, device)
    decls = declared_tensors(arch, config, compute, stored_names=list(source.entries))
    source.choose_prefix(decls)
    source.check(decls)
    with torch.no_grad():
        return arch.build(config, source)


def build_random_model(config, seed: int, dtype="bfloat16", device="cuda:0", std: float = 0.02,
                       norm_std: float = 0.1, architecture: Optional[str] = None):
    """A model with seeded random weights made on the device (no file)."""
    arch = get_architecture(architecture or config.architecture)
    source = RandomWeights(seed, parse_dtype(dtype), device, std=std, norm_std=norm_std)
    with torch.no_grad():
        return arch.build(config, source)


def write_random_model(config: Union[dict, object], out_dir: str, seed: int, std: float = 0.02,
                       norm_std: float = 0.1, store_dtype="bfloat16", architecture: Optional[str] = None) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` with seeded random weights:
    ``N(0, std)`` for matrices and routers, ``1 + N(0, norm_std)`` for norm weights, drawn in
    float32 from one CPU generator in declaration order and stored as ``store_dtype``."""
    if isinstance(config, dict):
        arch, typed = resolve(config, "config")
    else:
        arch, typed = get_architecture(architecture or config.architecture), config
    store = parse_dtype(store_dtype)
    os.makedirs(out_dir, exist_ok=True)
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    tensors = []
    for d in declared_tensors(arch, typed):
        if d.role == "table":
            t = torch.zeros(d.shape, dtype=torch.int32)
        else:
            t = torch.randn(d.shape, generator=gen, dtype=torch.float32)
            t = (1.0 + norm_std * t) if d.init == "norm" else std * t
            t = t.to(store)
        tensors.append((d.name, t))
    safetensors_io.save_file(tensors, os.path.join(out_dir, "model.safetensors"),
                             metadata={"format": "pt", "seed": str(seed)})
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(typed.to_dict(), fh, indent=2)
    return out_dir
