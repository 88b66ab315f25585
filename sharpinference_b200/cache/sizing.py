"""How many pages each cache group gets out of a memory budget.

A group whose mask forgets the past (chunk, window) never holds more of a request than the span it
can still see plus the portion being written: pages below that are given back after every step.
Such groups are sized for ``max_batch`` requests at that bound; what is left of the budget goes to
the groups that keep every position (full), which all hold the same positions and therefore get
the same number of pages.  The reference sizes one contiguous cache per sequence from its context
length (src/SharpInference.Engine/CudaSequenceKvCache.cs:20-58); with a shared pool the question
is how to split it.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

MAX_GROUP_TOKENS = 1 << 22


def group_layout(schedule: Sequence, blocks: Sequence) -> List[Tuple[object, int]]:
    """``(cache spec, number of schedule entries that write it)`` per group, in the order in which
    :class:`CacheManager` numbers the groups."""
    order: List[object] = []
    count = {}
    for entry in schedule:
        spec = getattr(blocks[entry.layer].mixer, "cache_spec", None)
        if spec is None or entry.cache_from is not None:
            continue
        if spec not in count:
            order.append(spec)
            count[spec] = 0
        count[spec] += 1
    return [(spec, count[spec]) for spec in order]


def pages_per_group(groups: Sequence[Tuple[object, int]], *, budget_bytes: int, itemsize: int, page_size: int,
                    max_batch: int, max_tokens_per_step: int) -> List[int]:
    """Pages for every group of ``group_layout`` under ``budget_bytes``."""
    if not groups:
        return []

    def up(n: int) -> int:
        return (n + page_size - 1) // page_size * page_size

    per_token = [2 * spec.num_kv_heads * spec.head_dim * itemsize * entries for spec, entries in groups]
    bounded = [spec.kind != "full" for spec, _ in groups]
    # what a forgetting group can hold at most: per request its span, the portion in flight and the page that
    # straddles the edge
    cap = [min(MAX_GROUP_TOKENS, max_batch * (up(spec.span) + up(max_tokens_per_step) + page_size)) if b else 0
           for (spec, _), b in zip(groups, bounded)]
    tokens = [0] * len(groups)
    full = [i for i, b in enumerate(bounded) if not b]
    want = sum(cap[i] * per_token[i] for i in range(len(groups)) if bounded[i])
    # with full groups beside them the forgetting groups take at most half of the budget
    share = budget_bytes if not full else budget_bytes // 2
    scale = min(1.0, share / want) if want > 0 else 1.0
    spent = 0
    for i in range(len(groups)):
        if bounded[i]:
            tokens[i] = max(page_size, int(cap[i] * scale))
            spent += tokens[i] * per_token[i]
    if full:
        each = max(0, budget_bytes - spent) // max(1, sum(per_token[i] for i in full))
        for i in full:
            tokens[i] = max(page_size, min(MAX_GROUP_TOKENS, each))
    return [max(1, t // page_size) for t in tokens]
