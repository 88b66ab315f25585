"""Small stand-ins for the tests that need no GPU: blocks with only a cache need, a step
function that returns canned logits."""
from __future__ import annotations

from types import SimpleNamespace
from typing import List, Optional

import torch

from sharpinference_b200.cache import CacheManager
from sharpinference_b200.models.model import ScheduleEntry
from sharpinference_b200.parts.base import CacheSpec, StateSpec


def fake_blocks(specs: List[Optional[CacheSpec]], states: Optional[List[Optional[StateSpec]]] = None):
    states = states or [None] * len(specs)
    return [SimpleNamespace(mixer=SimpleNamespace(cache_spec=s, state_spec=st)) for s, st in zip(specs, states)]


def llama_like_manager(num_pages=8, page_size=4, chunk=8, max_requests=4, layers=4, nope=(3,), allocate=False,
                       device="cpu"):
    """Two groups as in Llama 4: chunked layers and full layers."""
    specs = [CacheSpec("full", 0, 2, 8) if i in nope else CacheSpec("chunk", chunk, 2, 8) for i in range(layers)]
    blocks = fake_blocks(specs)
    schedule = [ScheduleEntry(i) for i in range(layers)]
    return CacheManager(schedule, blocks, page_size=page_size, num_pages=num_pages, max_requests=max_requests,
                        dtype=torch.float32, device=device, allocate=allocate)
