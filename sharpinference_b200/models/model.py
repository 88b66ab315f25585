"""``DecoderModel``: embedding, a schedule of blocks, final norm and output head.

The schedule is data: a list of entries that name the block to run and, optionally, an earlier
entry whose cache this one reads instead of writing its own.  A block may be named more than
once (its weights are shared; each entry has a cache of its own unless it borrows one).  The
reference's precedent for borrowing is its key/value sharing between layers
(src/SharpInference.Engine/CudaSequenceKvCache.cs:25-33); its layer loop is fixed,
``for layer in 0..L`` (src/SharpInference.Engine/ForwardPass.cs:1539-1730).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from ..kernels import ops
from ..parts.base import Block, Norm, StepContext
from ..parts.linear import Linear


@dataclass(frozen=True)
class ScheduleEntry:
    layer: int                          # index into DecoderModel.blocks
    cache_from: Optional[int] = None    # schedule index whose cache this entry reads (no write of its own)


class DecoderModel:
    def __init__(self, *, embedding: torch.Tensor, blocks: Sequence[Block], final_norm: Norm, head: Linear,
                 act_dtype: torch.dtype, schedule: Optional[Sequence[ScheduleEntry]] = None,
                 eos_token_ids: Sequence[int] = (), config=None):
        self.embedding = embedding                  # [V, H]
        self.blocks: List[Block] = list(blocks)
        self.final_norm = final_norm
        self.head = head
        self.act_dtype = act_dtype
        self.schedule: List[ScheduleEntry] = (list(schedule) if schedule is not None
                                              else [ScheduleEntry(i) for i in range(len(self.blocks))])
        self.vocab_size, self.hidden_size = embedding.shape
        self.eos_token_ids = tuple(eos_token_ids)
        self.config = config
        self._validate_schedule()

    def set_schedule(self, schedule: Sequence[ScheduleEntry]) -> "DecoderModel":
        """Replace the order in which blocks run (before a cache manager is made for the model)."""
        self.schedule = list(schedule)
        self._validate_schedule()
        return self

    def _validate_schedule(self) -> None:
        for i, e in enumerate(self.schedule):
            if not (0 <= e.layer < len(self.blocks)):
                raise ValueError(f"schedule entry {i} names block {e.layer}; the model has {len(self.blocks)}")
            if e.cache_from is not None:
                if not (0 <= e.cache_from < i):
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_from}, which must come earlier")
                src = self.schedule[e.cache_from]
                if src.cache_from is not None:
                    raise ValueError(f"schedule entry {i} reads entry {e.cache_from}, which itself borrows a cache")
                a = self.blocks[e.layer].mixer.cache_spec
                b = self.blocks[src.layer].mixer.cache_spec
                if a is None or b is None or a != b:
                    raise ValueError(f"schedule entry {i} cannot read the cache of entry {e.cache_from}: "
                                     f"their cache needs differ ({a} against {b})")

    def forward(self, ctx: StepContext) -> Optional[torch.Tensor]:
        """Run the step's rows through every scheduled block; float32 logits ``[R, V]`` at
        ``ctx.want_rows`` (None if no logits are wanted)."""
        x = ops.embed_gather(ctx.token_ids, self.embedding)
        pending = None
        norms = ctx.extras.get("layer_norms")        # tracing: see StepRunner.trace_layers
        for index, entry in enumerate(self.schedule):
            x, pending = self.blocks[entry.layer].forward(ctx, ctx.slots[index], x, pending)
            if norms is not None:
                after = x.float() if pending is None else x.float() + pending.float()
                norms.append(after.square().sum(dim=1).sqrt())
        if ctx.want_rows is None or ctx.want_rows.numel() == 0:
            return None
        h, _ = self.final_norm.apply(x, pending, rows=ctx.want_rows, out_dtype=self.act_dtype)
        return self.head(h)
