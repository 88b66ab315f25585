"""The step function: one batch of (request, its next tokens) through the model, from the cache.

A step's entries are portions of prompts beside single decoded tokens, cut anywhere.  The
function runs exactly the rows it is given, as one batch: the rows of all entries are laid end
to end (no padding), every row knows its absolute position and its request, attention reads
earlier positions from the request's pages, and float32 logits come back for the rows that were
asked for, in entry order.

The reference has two separate calls that are never mixed and that refuse mixture-of-experts
models: ``PrefillPackedMulti`` (portions of several prompts as packed rows,
src/SharpInference.Engine/ForwardPass.cs:2727-2916) and ``BatchForwardMulti`` (one token per
sequence, :2551-2703); both append keys and values first and advance lengths only after the
pass (:2880-2882).  The same holds here: pages are reserved before the launch, lengths are
committed after it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..kernels import ops
from ..parts.base import StepContext


class StepError(ValueError):
    """A step that cannot run as given (unknown request, bad token id, bad wanted place)."""


@dataclass
class StepEntry:
    request_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)   # places among `tokens` whose logits are wanted


class StepRunner:
    ATTENTION_TILE = 64        # rows of one request that one attention CTA serves
    DECODE_ROWS_UP_TO = 4      # entries this short are served row by row by the split-KV kernel

    def __init__(self, model, cache: CacheManager):
        self.model = model
        self.cache = cache
        self.device = cache.device
        self._slots = cache.layer_slots()
        self.steps_run = 0
        self.rows_run = 0
        # Tracing, for hunting the first difference: when `trace_router` is set, every routed
        # feed-forward of a step leaves the expert it chose per row in `last_router_choices`
        # (one int32 [T] tensor per routed schedule entry, in schedule order).  The reference
        # prints the same with SHARPI_TRACE_ROUTERS (src/SharpInference.Engine/ForwardPass.cs:2042-2056).
        self.trace_router = False
        # after every step, read the word in which a tensor-core kernel records a wait that gave up
        # (a 4-byte copy; the step's result is read by the host right after anyway)
        self.check_kernel_status = True
        self.last_router_choices: List[torch.Tensor] = []

    def validate(self, entries: Sequence[StepEntry]) -> None:
        """Refuse, before any page is taken, a step that cannot run as given."""
        if not entries:
            raise StepError("a step needs at least one entry")
        V = self.model.vocab_size
        seen = set()
        for e in entries:
            if e.request_id in seen:
                raise StepError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            if e.request_id not in self.cache.requests:
                raise StepError(f"request {e.request_id!r} is not live")
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {e.request_id!r}: an entry must bring at least one token")
            for w in e.want:
                if not (0 <= w < n):
                    raise StepError(f"request {e.request_id!r}: wanted place {w} is outside its {n} token(s)")
            for t in e.tokens:
                if not (0 <= t < V):
                    raise StepError(f"token id {t} is outside the vocabulary [0, {V})")

    def build_context(self, entries: Sequence[StepEntry]) -> StepContext:
        """Lay out the step's metadata: one pinned host buffer, one copy to the device."""
        cache = self.cache
        starts, lengths, slots = [], [], []
        for e in entries:
            rc = cache.get(e.request_id)
            starts.append(rc.length)
            lengths.append(len(e.tokens))
            slots.append(rc.state_slot)
        B = len(entries)
        T = sum(lengths)
        tokens = np.empty(T, dtype=np.int64)
        positions = np.empty(T, dtype=np.int32)
        row_request = np.empty(T, dtype=np.int32)
        row_offsets = np.zeros(B + 1, dtype=np.int32)
        want_rows: List[int] = []
        tiles: List[int] = []            # (first row, rows, first position, request) per attention tile
        decode_rows: List[int] = []
        r = 0
        for b, e in enumerate(entries):
            n = lengths[b]
            if n <= self.DECODE_ROWS_UP_TO:
                decode_rows.extend(range(r, r + n))
            else:
                for t0 in range(0, n, self.ATTENTION_TILE):
                    tiles.extend((r + t0, min(self.ATTENTION_TILE, n - t0), starts[b] + t0, b))
            tokens[r:r + n] = np.asarray(e.tokens, dtype=np.int64)
            positions[r:r + n] = np.arange(starts[b], starts[b] + n, dtype=np.int32)
            row_request[r:r + n] = b
            want_rows.extend(r + w for w in e.want)
            r += n
            row_offsets[b + 1] = r

        # Block tables, one per group, padded to a common width with -1.
        ids = [e.request_id for e in entries]
        width = 1
        for g in cache.groups:
            for rid in ids:
                width = max(width, len(cache.requests[rid].tables[g.index]))
        G = len(cache.groups)
        R = len(want_rows)
        # layout of the one int32 staging buffer
        n_tiles, n_dec = len(tiles) // 4, len(decode_rows)
        sizes = [T, T, T, B, B + 1, B, R] + [B * width] * G + [4 * n_tiles, n_dec]
        offsets = np.concatenate([[0], np.cumsum([(s + 3) // 4 * 4 for s in sizes])])
        host = torch.empty(int(offsets[-1]), dtype=torch.int32, pin_memory=self.device.type == "cuda")
        hv = host.numpy()
        hv[offsets[0]:offsets[0] + T] = tokens
        hv[offsets[1]:offsets[1] + T] = positions
        hv[offsets[2]:offsets[2] + T] = row_request
        hv[offsets[3]:offsets[3] + B] = starts
        hv[offsets[4]:offsets[4] + B + 1] = row_offsets
        hv[offsets[5]:offsets[5] + B] = slots
        hv[offsets[6]:offsets[6] + R] = want_rows
        for gi, g in enumerate(cache.groups):
            table = np.full((B, width), -1, dtype=np.int32)
            for b, rid in enumerate(ids):
                t = cache.requests[rid].tables[g.index]
                table[b, :len(t)] = t
            o = offsets[7 + gi]
            hv[o:o + B * width] = table.reshape(-1)
        hv[offsets[7 + G]:offsets[7 + G] + 4 * n_tiles] = tiles
        hv[offsets[8 + G]:offsets[8 + G] + n_dec] = decode_rows
        dev = host.to(self.device, non_blocking=True)

        def view(i: int, n: int) -> torch.Tensor:
            return dev[int(offsets[i]):int(offsets[i]) + n]

        return StepContext(
            num_tokens=T, num_requests=B, token_ids=view(0, T), positions=view(1, T), row_request=view(2, T),
            request_start=view(3, B), row_offsets=view(4, B + 1), state_slots=view(5, B),
            block_tables={g.index: view(7 + gi, B * width).view(B, width) for gi, g in enumerate(cache.groups)},
            want_rows=view(6, R) if R else None, slots=self._slots,
            host_starts=starts, host_lengths=lengths, host_state_slots=slots,
            max_rows_per_request=max(lengths), max_context=max(s + n for s, n in zip(starts, lengths)),
            decode_only=all(n == 1 for n in lengths),
            attn_tiles=view(7 + G, 4 * n_tiles).view(n_tiles, 4) if n_tiles else None, num_attn_tiles=n_tiles,
            decode_rows=view(8 + G, n_dec) if (n_dec and n_dec != T) else None, num_decode_rows=n_dec,
        )

    @torch.no_grad()
    def run(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run one step.  Returns float32 logits ``[wanted, vocab]`` on the device, in the order of
        the entries and of each entry's ``want`` (None if nothing was wanted).  Raises
        :class:`OutOfPages` before anything ran if the pages for the step cannot all be had."""
        self.validate(entries)
        self.cache.reserve([(e.request_id, len(e.tokens)) for e in entries])
        ctx = self.build_context(entries)
        if self.trace_router:
            ctx.extras["router_choices"] = []
        logits = self.model.forward(ctx)
        if self.check_kernel_status:
            ops.check_status(self.device)
        self.last_router_choices = ctx.extras.get("router_choices", [])
        for e in entries:
            self.cache.commit(e.request_id, len(e.tokens))
        self.steps_run += 1
        self.rows_run += ctx.num_tokens
        return logits
