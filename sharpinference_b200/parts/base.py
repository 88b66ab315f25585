"""Interfaces of the parts a layer is put together from, and the step context they run in.

A decoder layer here is a *block* that arranges a *mixer* (attention, or anything else that
moves information between positions), a *feed-forward*, *norms* and, inside the mixer, a
*position encoding*.  Every part receives its sizes and constants as constructor arguments and
its tensors from a weight source; no part knows which model it is in.  The reference decides
the same questions with per-architecture flags inside one forward pass
(src/SharpInference.Engine/ForwardPass.cs:1534-1757, flags from
src/SharpInference.Core/ModelGraph.cs:262-347); here they are parts chosen layer by layer.

Adding a part: subclass the interface below, give it a ``kind`` name with
:func:`register_part`, and use it from an architecture's builder (or a test's).  Contracts:

``Mixer.forward(ctx, slot, h) -> [T, H] float32``
    ``h`` are the normalised activations of the step's T rows in the activation dtype.
    ``slot`` is the cache manager's grant for this place in the layer schedule: the pages of its
    cache group (if ``cache_spec`` is not None) and the per-request state (if ``state_spec`` is
    not None).  The result is added to the residual stream by the block.
``FeedForward.forward(ctx, h, h32) -> [T, H] float32``
    ``h32`` is the unrounded float32 copy of ``h``, given when ``wants_fp32_input`` is true.
``Norm.apply(x, delta, rows, out_dtype, want_fp32) -> (h, h32)``
    ``x`` is the float32 residual stream; ``delta`` (float32 or None) is added to it first.
``PositionEncoding``
    either describes a rotation the attention kernel applies itself (``rotary()``), or edits q
    and k in place through ``apply(ctx, q, k)``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from types import SimpleNamespace
from typing import Any, Callable, Dict, Hashable, List, Optional, Sequence, Tuple

import torch


# ---------------------------------------------------------------------------------------
# What a mixer needs from the cache manager
# ---------------------------------------------------------------------------------------
@dataclass(frozen=True)
class CacheSpec:
    """Keys and values a mixer keeps per position, and which past positions stay visible.

    ``kind`` is ``"full"`` (every earlier position), ``"chunk"`` (positions of the same chunk of
    ``span`` positions) or ``"window"`` (the last ``span`` positions, the query's own included).
    Layers with equal specs share one group of pages and one block table per request.
    """

    kind: str
    span: int
    num_kv_heads: int
    head_dim: int

    def __post_init__(self):
        if self.kind not in ("full", "chunk", "window"):
            raise ValueError(f"cache kind '{self.kind}' is not one of full, chunk, window")
        if self.kind != "full" and self.span <= 0:
            raise ValueError(f"cache kind '{self.kind}' needs a positive span, found {self.span}")

    def lowest_visible(self, pos: int) -> int:
        """The lowest position a query at ``pos`` may read."""
        if self.kind == "chunk":
            return (pos // self.span) * self.span
        if self.kind == "window":
            return max(0, pos - self.span + 1)
        return 0


@dataclass(frozen=True)
class StateSpec:
    """A tensor of fixed shape that a mixer keeps for every live request."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class LayerSlot:
    """What one entry of the layer schedule was granted by the cache manager."""

    index: int                              # place in the schedule
    layer: int                              # which block runs there
    group: Optional[int] = None             # id of the page group (key of StepContext.block_tables)
    kv: Optional[torch.Tensor] = None       # [pages, 2, kv_heads, page_size, head_dim]
    writes_cache: bool = True               # False: reads the cache that another entry writes
    state: Optional[torch.Tensor] = None    # [state_slots, *StateSpec.shape]
    page_size: int = 0


@dataclass
class StepContext:
    """One step's batch, as the parts see it.  Device tensors are int32."""

    num_tokens: int
    num_requests: int
    token_ids: torch.Tensor                 # [T]
    positions: torch.Tensor                 # [T] absolute position of every row
    row_request: torch.Tensor               # [T] index of the row's request within this step
    request_start: torch.Tensor             # [B] position of the request's first row in this step
    row_offsets: torch.Tensor               # [B + 1] first row of every request
    state_slots: torch.Tensor               # [B] state slot of every request
    block_tables: Dict[int, torch.Tensor]   # group id -> [B, max_blocks] page ids (-1: none)
    want_rows: Optional[torch.Tensor]       # [R] rows whose logits are wanted (None: no logits)
    slots: List[LayerSlot]                  # one per schedule entry
    # host-side copies, for grid sizing and for parts written in plain torch
    host_starts: List[int] = field(default_factory=list)
    host_lengths: List[int] = field(default_factory=list)
    host_state_slots: List[int] = field(default_factory=list)
    max_rows_per_request: int = 0
    max_context: int = 0                    # highest position + 1 over the step (an upper bound in a replayed graph)
    decode_only: bool = False               # every request brings exactly one row
    # what the mixers' step planners made of this step, by planner key: the arrays as int32 device tensors
    # (None where an array is empty) and the host-side values, as attributes (see StepPlanner)
    plans: Dict[Hashable, SimpleNamespace] = field(default_factory=dict)
    extras: Dict[str, Any] = field(default_factory=dict)


# ---------------------------------------------------------------------------------------
# Per-step metadata that a kind of mixer brings along
# ---------------------------------------------------------------------------------------
@dataclass
class StepPlanData:
    """What a planner made of one step: int32 host arrays (any shape) that travel to the device in the
    step's one metadata copy, and host-side values (counts, bounds) that the mixer's launches use."""

    arrays: Dict[str, Any] = field(default_factory=dict)
    values: Dict[str, Any] = field(default_factory=dict)


class StepPlanner:
    """How a kind of mixer cuts a step's rows for its kernels.

    The step function knows requests, rows and block tables; how a mixer's kernels want the rows grouped
    (tiles of a prompt portion, single rows, segments of a scan) is the mixer's business.  A mixer that needs
    such metadata returns a planner from ``Mixer.step_planner(page_size)``.  Planners with equal ``key`` are
    one planner: they run once per step and every mixer with that key reads ``ctx.plans[key]``.

    ``plan(starts, lengths, bucket)`` gets, per request of the step, the position of its first row and its
    number of rows (rows of all requests lie end to end).  For decode-only steps that are replayed as a CUDA
    graph, ``bucket(starts, lengths)`` names what of the plan is baked into the graph (grid sizes, bounds):
    steps with the same number of requests and the same bucket share a graph, and ``plan`` is then called
    with that bucket and must return arrays of the same shapes, and values that hold for every such step.
    """

    key: Hashable = None

    def plan(self, starts: Sequence[int], lengths: Sequence[int], bucket: Hashable = None) -> StepPlanData:
        raise NotImplementedError

    def bucket(self, starts: Sequence[int], lengths: Sequence[int]) -> Hashable:
        return None


# ---------------------------------------------------------------------------------------
# Part interfaces
# ---------------------------------------------------------------------------------------
class Part:
    kind: str = ""


class Norm(Part):
    def apply(self, x: torch.Tensor, delta: Optional[torch.Tensor], *, rows: Optional[torch.Tensor],
              out_dtype: torch.dtype, want_fp32: bool = False):
        raise NotImplementedError


class PositionEncoding(Part):
    def rotary(self) -> Optional[Tuple[torch.Tensor, str]]:
        """``(inv_freq float32 [head_dim / 2], pairing)`` with pairing ``"interleaved"`` (pairs
        ``(2j, 2j+1)``) or ``"halves"`` (pairs ``(j, j + d/2)``) if the encoding is a rotation by
        ``position * inv_freq``; None otherwise."""
        return None

    def apply(self, ctx: StepContext, q: torch.Tensor, k: torch.Tensor) -> None:
        """Edit ``q`` [T, heads, d] and ``k`` [T, kv_heads, d] (float32) in place."""
        raise NotImplementedError


class Mixer(Part):
    cache_spec: Optional[CacheSpec] = None
    state_spec: Optional[StateSpec] = None

    def step_planner(self, page_size: int) -> Optional[StepPlanner]:
        """The planner of this mixer's per-step metadata, or None if the step context is all it needs."""
        return None

    def forward(self, ctx: StepContext, slot: LayerSlot, h: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    wants_fp32_input: bool = False

    def forward(self, ctx: StepContext, h: torch.Tensor, h32: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    mixer: Mixer

    def forward(self, ctx: StepContext, slot: LayerSlot, x: torch.Tensor, pending: Optional[torch.Tensor]):
        """Returns ``(x, pending)``: the residual stream and a float32 update not yet added to it
        (the next norm adds it, fused)."""
        raise NotImplementedError


# ---------------------------------------------------------------------------------------
# Registry of part kinds
# ---------------------------------------------------------------------------------------
_PARTS: Dict[str, Dict[str, Callable[..., Part]]] = {
    "norm": {}, "position": {}, "mixer": {}, "feed_forward": {}, "block": {},
}


def register_part(category: str, kind: str):
    """Class decorator: make ``kind`` constructible through :func:`make_part`."""
    if category not in _PARTS:
        raise ValueError(f"unknown part category '{category}' (known: {', '.join(_PARTS)})")

    def deco(cls):
        cls.kind = kind
        _PARTS[category][kind] = cls
        return cls

    return deco


def make_part(category: str, kind: str, **params) -> Part:
    try:
        cls = _PARTS[category][kind]
    except KeyError:
        known = ", ".join(sorted(_PARTS.get(category, {}))) or "(none)"
        raise ValueError(f"no {category} part of kind '{kind}' is registered; known: {known}") from None
    return cls(**params)


def part_kinds(category: str) -> List[str]:
    return sorted(_PARTS[category])
