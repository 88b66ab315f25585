"""Where a model builder gets its tensors from.

A builder (see :mod:`sharpinference_b200.registry`) asks a ``WeightSource`` for every tensor by
the name it has in the file, with the shape it must have:

``matrix(name, shape)``
    an operand of a matrix product.  It is kept in bfloat16; a tensor stored in 32-bit stays
    32-bit; under ``dtype=float32`` everything becomes float32.
``vector(name, shape, init=...)``
    a small tensor used in 32-bit arithmetic (norm weights, the router): always float32.
``table(name, shape)``
    an integer table: int32.

Three sources implement it: :class:`DeclaringWeights` (no data: records what a model needs, on
the ``meta`` device), :class:`FileWeights` (safetensors, checked against the declaration first
so that one error lists every missing, unexpected and misshaped tensor) and
:class:`RandomWeights` (seeded normal draws made on the device, for benchmarks whose weights
would not fit a file comfortably).

The reference resolves every tensor once in the forward pass's constructor and throws
"Missing tensor: name" on the first miss (src/SharpInference.Engine/ForwardPass.cs:289-413,
:2301-2306); its shape check reads "tensor 'x' has shape [...], expected [...]"
(src/SharpInference.Engine/DSparkHostHeads.cs:163-170).
"""
from __future__ import annotations

import zlib
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import safetensors_io


class WeightError(ValueError):
    """Tensors of a model folder do not match what the architecture needs."""


@dataclass(frozen=True)
class TensorDecl:
    name: str
    shape: Tuple[int, ...]
    role: str          # "matrix" | "vector" | "table"
    init: str          # "normal" | "norm" | "zeros"


class WeightSource:
    compute_dtype: torch.dtype = torch.bfloat16
    device: torch.device = torch.device("cpu")

    def matrix(self, name: str, shape: Sequence[int]) -> torch.Tensor:
        raise NotImplementedError

    def vector(self, name: str, shape: Sequence[int], init: str = "norm") -> torch.Tensor:
        raise NotImplementedError

    def table(self, name: str, shape: Sequence[int]) -> torch.Tensor:
        raise NotImplementedError

    def has(self, name: str) -> bool:
        """Whether an optional tensor is there (a declaring source answers for the layout it declares)."""
        return True

    def stored(self, name: str) -> Optional[bool]:
        """Whether a folder holds ``name``: for builders that accept two layouts of the same weights and must
        ask for the one that is there.  None where there is no folder to look into (random weights, a bare
        declaration): the builder then takes its first layout."""
        return None


class DeclaringWeights(WeightSource):
    """Hands out shape-only tensors and remembers what was asked for."""

    def __init__(self, compute_dtype: torch.dtype = torch.bfloat16, optional_present: bool = True,
                 stored_names: Optional[Sequence[str]] = None, prefixes: Sequence[str] = ("",)):
        self.compute_dtype = compute_dtype
        self.device = torch.device("meta")
        self.decls: List[TensorDecl] = []
        self._names: Dict[str, TensorDecl] = {}
        self._optional_present = optional_present
        # the names a folder holds, when the declaration is made to check that folder
        self._stored = None if stored_names is None else set(stored_names)
        self._prefixes = tuple(prefixes)

    def stored(self, name):
        if self._stored is None:
            return None
        return any(pre + name in self._stored for pre in self._prefixes)

    def _declare(self, name: str, shape: Sequence[int], role: str, init: str, dtype: torch.dtype) -> torch.Tensor:
        decl = TensorDecl(name, tuple(int(s) for s in shape), role, init)
        prev = self._names.get(name)
        if prev is None:
            self._names[name] = decl
            self.decls.append(decl)
        elif prev.shape != decl.shape:
            raise WeightError(f"tensor '{name}' is asked for with two shapes: {list(prev.shape)} and {list(decl.shape)}")
        return torch.empty(decl.shape, dtype=dtype, device="meta")

    def matrix(self, name, shape):
        return self._declare(name, shape, "matrix", "normal", self.compute_dtype)

    def vector(self, name, shape, init="norm"):
        return self._declare(name, shape, "vector", init, torch.float32)

    def table(self, name, shape):
        return self._declare(name, shape, "table", "zeros", torch.int32)

    def has(self, name):
        return self._optional_present


class FileWeights(WeightSource):
    """Tensors of a model folder, moved to ``device`` in the dtype the role asks for."""

    def __init__(self, model_dir: str, compute_dtype: torch.dtype, device, prefix: Optional[str] = None):
        self.compute_dtype = compute_dtype
        self.device = torch.device(device)
        self.model_dir = model_dir
        self.entries = safetensors_io.open_model(model_dir)
        self.prefix = prefix if prefix is not None else ""

    def stored(self, name):
        return self.prefix + name in self.entries

    # -- checking ----------------------------------------------------------------------
    def choose_prefix(self, decls: Sequence[TensorDecl], candidates=("", "language_model.")) -> str:
        """Checkpoints of a multimodal model keep the text model under ``language_model.``."""
        best, best_hits = "", -1
        for cand in candidates:
            hits = sum(1 for d in decls if cand + d.name in self.entries)
            if hits > best_hits:
                best, best_hits = cand, hits
        self.prefix = best
        return best

    def check(self, decls: Sequence[TensorDecl]) -> None:
        """Raise one ``WeightError`` listing every missing, misshaped, unsupported and unexpected tensor."""
        missing, wrong, unsupported = [], [], []
        wanted = set()
        for d in decls:
            full = self.prefix + d.name
            wanted.add(full)
            entry = self.entries.get(full)
            if entry is None:
                missing.append(f"{full}  expected shape {list(d.shape)}")
                continue
            if tuple(entry.shape) != d.shape:
                wrong.append(f"tensor '{full}' has shape {list(entry.shape)}, expected {list(d.shape)}")
            ok = ("F32", "BF16", "F16") if d.role != "table" else ("I32", "I64", "I16", "I8", "U8")
            if entry.dtype_name not in ok:
                unsupported.append(f"tensor '{full}' has dtype {entry.dtype_name}; a {d.role} takes {', '.join(ok)}")
        unexpected = sorted(n for n in self.entries if n not in wanted and n.startswith(self.prefix))
        if missing or wrong or unsupported or unexpected:
            parts = [f"{self.model_dir}: the tensors do not match the architecture"]
            for title, items in (("missing", missing), ("wrong shape", wrong), ("unsupported dtype", unsupported),
                                 ("unexpected", unexpected)):
                if items:
                    parts.append(f"  {title} ({len(items)}):")
                    parts.extend(f"    {i}" for i in items)
            raise WeightError("\n".join(parts))

    # -- loading -----------------------------------------------------------------------
    def _load(self, name: str, shape: Sequence[int]) -> torch.Tensor:
        full = self.prefix + name
        entry = self.entries.get(full)
        if entry is None:
            raise WeightError(f"Missing tensor: {full}")
        if tuple(entry.shape) != tuple(shape):
            raise WeightError(f"tensor '{full}' has shape {list(entry.shape)}, expected {list(shape)}")
        return entry.load().to(self.device, non_blocking=False)

    def matrix(self, name, shape):
        t = self._load(name, shape)
        if self.compute_dtype == torch.float32 or t.dtype == torch.float32:
            return t.to(torch.float32)
        return t.to(torch.bfloat16)

    def vector(self, name, shape, init="norm"):
        return self._load(name, shape).to(torch.float32)

    def table(self, name, shape):
        return self._load(name, shape).to(torch.int32)

    def has(self, name):
        return self.prefix + name in self.entries


class RandomWeights(WeightSource):
    """Seeded normal draws made directly on ``device``: ``N(0, std)`` for matrices and routers,
    ``1 + N(0, norm_std)`` for norm weights, as if they had been stored in ``store_dtype``."""

    def __init__(self, seed: int, compute_dtype: torch.dtype, device, std: float = 0.02, norm_std: float = 0.1,
                 store_dtype: torch.dtype = torch.bfloat16):
        self.seed = int(seed)
        self.compute_dtype = compute_dtype
        self.device = torch.device(device)
        self.std, self.norm_std, self.store_dtype = float(std), float(norm_std), store_dtype

    def _gen(self, name: str) -> torch.Generator:
        g = torch.Generator(device=self.device)
        g.manual_seed((self.seed * 1000003 + zlib.crc32(name.encode("utf-8"))) & 0x7FFFFFFFFFFFFFFF)
        return g

    def _draw(self, name: str, shape, std: float, mean: float) -> torch.Tensor:
        t = torch.empty(tuple(shape), dtype=self.store_dtype, device=self.device)
        t.normal_(mean, std, generator=self._gen(name)) if std > 0 else t.fill_(mean)
        return t

    def matrix(self, name, shape):
        t = self._draw(name, shape, self.std, 0.0)
        if self.compute_dtype == torch.float32 or t.dtype == torch.float32:
            return t.to(torch.float32)
        return t.to(torch.bfloat16)

    def vector(self, name, shape, init="norm"):
        if init == "norm":
            return self._draw(name, shape, self.norm_std, 1.0).to(torch.float32)
        return self._draw(name, shape, self.std, 0.0).to(torch.float32)

    def table(self, name, shape):
        return torch.zeros(tuple(shape), dtype=torch.int32, device=self.device)
