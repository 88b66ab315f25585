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
from types import SimpleNamespace
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..kernels import library, ops
from ..parts.base import StepContext


class StepError(ValueError):
    """A step that cannot run as given (unknown request, bad token id, bad wanted place).  ``request_id``
    names the entry at fault when there is one; nothing was reserved or launched."""

    def __init__(self, message: str, request_id: Hashable = None):
        super().__init__(message)
        self.request_id = request_id


@dataclass
class StepEntry:
    request_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)   # places among `tokens` whose logits are wanted


@dataclass
class HostStep:
    """One step's metadata laid out on the host: the int32 words of the staging buffer, where each named
    segment lies in it (offset, shape), and what the planners returned beside their arrays."""

    words: np.ndarray
    segments: Dict[object, tuple]                    # name -> (offset in words, shape)
    plan_values: Dict[Hashable, dict]
    starts: List[int]
    lengths: List[int]
    slots: List[int]
    num_wanted: int
    width: int


class StepRunner:
    def __init__(self, model, cache: CacheManager):
        self.model = model
        self.cache = cache
        self.device = cache.device
        self._slots = cache.layer_slots()
        # Mixers that cut the step's rows for their kernels bring a planner (parts.base.StepPlanner); planners
        # with equal keys are one.  The step function runs each once per step and ships its arrays in the
        # step's one metadata copy; it knows nothing of what they mean.
        self.planners: Dict[Hashable, object] = {}
        for b in getattr(model, "blocks", []):
            make = getattr(b.mixer, "step_planner", None)
            planner = make(cache.page_size) if make is not None else None
            if planner is not None:
                self.planners.setdefault(planner.key, planner)
        self.steps_run = 0
        self.rows_run = 0
        # Tracing, for hunting the first difference: when `trace_router` is set, every routed
        # feed-forward of a step leaves the expert it chose per row in `last_router_choices`
        # (one int32 [T] tensor per routed schedule entry, in schedule order).  The reference
        # prints the same with SHARPI_TRACE_ROUTERS (src/SharpInference.Engine/ForwardPass.cs:2042-2056).
        self.trace_router = False
        # `trace_layers`: after every scheduled block the L2 norm of every row of the residual stream, in
        # `last_layer_norms` (one float32 [T] tensor per schedule entry); the reference prints the same per
        # layer with SHARPI_TRACE_NORMS (src/SharpInference.Engine/ForwardPass.cs:1795-1819).  Traced steps
        # run eagerly, never as a replayed graph.
        self.trace_layers = False
        self.last_layer_norms: list = []
        # after every step, read the word in which a tensor-core kernel records a wait that gave up
        # (a 4-byte copy; the step's result is read by the host right after anyway)
        self.check_kernel_status = True
        self._status_host, self._status_event, self._status_pending = None, None, False
        self.last_router_choices: List[torch.Tensor] = []
        # Decode-only steps are launch-bound at small batches, so they are captured once per shape
        # (requests, wanted rows, block-table width, the planners' buckets) as a CUDA graph and replayed; the
        # step's metadata lives in one static device buffer that is refreshed before each replay.  The
        # reference does the same for its per-token decode (src/SharpInference.Engine/CudaForwardPass.cs:1668-1675).
        # Only models whose parts read the step through device tensors alone can be captured.
        self.use_graphs = all(getattr(b.mixer, "graph_safe", False) and getattr(getattr(b, "ffn", None), "graph_safe", False)
                              for b in model.blocks) if hasattr(model, "blocks") else False
        self.max_graphs = 32
        self._graphs: Dict[tuple, dict] = {}
        self._graph_seen: set = set()
        self._graph_pool = None
        self.graph_replays = 0

    def validate(self, entries: Sequence[StepEntry]) -> None:
        """Refuse, before any page is taken, a step that cannot run as given."""
        if not entries:
            raise StepError("a step needs at least one entry")
        V = self.model.vocab_size
        seen = set()
        for e in entries:
            if e.request_id in seen:
                raise StepError(f"request {e.request_id!r} appears twice in one step", e.request_id)
            seen.add(e.request_id)
            if e.request_id not in self.cache.requests:
                raise StepError(f"request {e.request_id!r} is not live", e.request_id)
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {e.request_id!r}: an entry must bring at least one token", e.request_id)
            for w in e.want:
                if not (0 <= w < n):
                    raise StepError(f"request {e.request_id!r}: wanted place {w} is outside its {n} token(s)",
                                    e.request_id)
            for t in e.tokens:
                if not (0 <= t < V):
                    raise StepError(f"request {e.request_id!r}: token id {t} is outside the vocabulary [0, {V})",
                                    e.request_id)

    def lay_out(self, entries: Sequence[StepEntry], width: Optional[int] = None,
                buckets: Optional[Dict[Hashable, Hashable]] = None) -> HostStep:
        """The step's metadata as one int32 array (every segment starting on 16 bytes): token ids, positions,
        row -> request, request starts, row offsets, state slots, wanted rows, one block table per cache
        group, then every planner's arrays.  ``width`` pads the block tables to a fixed number of columns;
        ``buckets`` (planner key -> bucket) is what a replayed graph fixed of each planner's plan."""
        cache = self.cache
        starts, lengths, slots = [], [], []
        for e in entries:
            rc = cache.get(e.request_id)
            starts.append(rc.length)
            lengths.append(len(e.tokens))
            slots.append(rc.state_slot)
        B, T = len(entries), sum(lengths)
        tokens = np.empty(T, dtype=np.int64)
        positions = np.empty(T, dtype=np.int32)
        row_request = np.empty(T, dtype=np.int32)
        row_offsets = np.zeros(B + 1, dtype=np.int32)
        want_rows: List[int] = []
        r = 0
        for b, e in enumerate(entries):
            n = lengths[b]
            tokens[r:r + n] = np.asarray(e.tokens, dtype=np.int64)
            positions[r:r + n] = np.arange(starts[b], starts[b] + n, dtype=np.int32)
            row_request[r:r + n] = b
            want_rows.extend(r + w for w in e.want)
            r += n
            row_offsets[b + 1] = r
        ids = [e.request_id for e in entries]
        needed = self.table_width(ids)
        if width is None:
            width = needed
        elif width < needed:
            raise StepError(f"block tables need {needed} columns, the buffer has {width}")
        pieces: List[tuple] = [("token_ids", tokens), ("positions", positions), ("row_request", row_request),
                               ("request_start", np.asarray(starts, dtype=np.int32)), ("row_offsets", row_offsets),
                               ("state_slots", np.asarray(slots, dtype=np.int32)),
                               ("want_rows", np.asarray(want_rows, dtype=np.int32))]
        for g in cache.groups:
            table = np.full((B, width), -1, dtype=np.int32)
            for b, rid in enumerate(ids):
                t = cache.requests[rid].tables[g.index]
                table[b, :len(t)] = t
            pieces.append((("table", g.index), table))
        plan_values: Dict[Hashable, dict] = {}
        for key, planner in self.planners.items():
            data = planner.plan(starts, lengths, None if buckets is None else buckets.get(key))
            plan_values[key] = dict(data.values)
            for name in sorted(data.arrays):
                pieces.append((("plan", key, name), np.ascontiguousarray(data.arrays[name], dtype=np.int32)))
        segments, at = {}, 0
        for name, arr in pieces:
            segments[name] = (at, tuple(arr.shape))
            at += (arr.size + 3) // 4 * 4
        words = np.zeros(at, dtype=np.int32)
        for name, arr in pieces:
            o = segments[name][0]
            words[o:o + arr.size] = arr.reshape(-1)
        return HostStep(words, segments, plan_values, starts, lengths, slots, len(want_rows), width)

    def build_context(self, entries: Sequence[StepEntry], width: Optional[int] = None,
                      buffers: Optional[tuple] = None, buckets: Optional[Dict[Hashable, Hashable]] = None,
                      host_step: Optional[HostStep] = None) -> StepContext:
        """Lay out the step's metadata and bring it to the device in one copy.  ``buffers`` = (pinned host
        tensor, device tensor) of exactly the layout's size are reused instead of fresh ones (graph replay)."""
        hs = host_step if host_step is not None else self.lay_out(entries, width, buckets)
        total = hs.words.size
        if buffers is None:
            host = torch.empty(total, dtype=torch.int32, pin_memory=self.device.type == "cuda")
        else:
            host = buffers[0]
            if host.numel() != total:
                raise StepError(f"static step buffer holds {host.numel()} words, this step needs {total}")
        host.numpy()[:] = hs.words
        if buffers is None:
            dev = host.to(self.device, non_blocking=True)
        else:
            dev = buffers[1]
            dev.copy_(host, non_blocking=True)

        def view(name) -> Optional[torch.Tensor]:
            o, shape = hs.segments[name]
            n = int(np.prod(shape)) if shape else 1
            return dev[o:o + n].view(shape) if n else None

        plans = {}
        for key in self.planners:
            fields = dict(hs.plan_values[key])
            for name in hs.segments:
                if isinstance(name, tuple) and name[0] == "plan" and name[1] == key:
                    fields[name[2]] = view(name)
            plans[key] = SimpleNamespace(**fields)
        B, T, lengths, starts = len(hs.lengths), sum(hs.lengths), hs.lengths, hs.starts
        return StepContext(
            num_tokens=T, num_requests=B, token_ids=view("token_ids"), positions=view("positions"),
            row_request=view("row_request"), request_start=view("request_start"), row_offsets=view("row_offsets"),
            state_slots=view("state_slots"),
            block_tables={g.index: view(("table", g.index)) for g in self.cache.groups},
            want_rows=view("want_rows"), slots=self._slots,
            host_starts=starts, host_lengths=lengths, host_state_slots=hs.slots,
            max_rows_per_request=max(lengths),
            # with a fixed table width the bound must hold for every later step that reuses the layout
            max_context=(max(s + n for s, n in zip(starts, lengths)) if buffers is None
                         else hs.width * self.cache.page_size),
            decode_only=all(n == 1 for n in lengths), plans=plans,
        )

    # The word in which a tensor-core kernel records a wait that gave up is copied to pinned host memory
    # behind every step and looked at when the next step begins (or when flush_status is called): by then
    # the caller has read the step's result, so the copy is there and nobody waits for it.  A kernel that
    # gave up therefore raises at the next step, or at the flush that ends a run.
    def _note_status(self) -> None:
        if self.device.type != "cuda":
            return
        if self._status_host is None:
            self._status_host = torch.zeros(1, dtype=torch.int32, pin_memory=True)
            self._status_event = torch.cuda.Event()
        self._status_host.copy_(ops.status_word(self.device), non_blocking=True)
        self._status_event.record()
        self._status_pending = True

    def flush_status(self) -> None:
        """Raise if a kernel of an earlier step gave up on a wait (waits for that step to finish)."""
        if not self._status_pending:
            return
        self._status_pending = False
        self._status_event.synchronize()
        if int(self._status_host[0]) != 0:
            ops.check_status(self.device)           # raises, and puts the word and the counters back to zero

    @torch.no_grad()
    def run(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run one step.  Returns float32 logits ``[wanted, vocab]`` on the device, in the order of
        the entries and of each entry's ``want`` (None if nothing was wanted).  Raises
        :class:`OutOfPages` before anything ran if the pages for the step cannot all be had."""
        self.flush_status()
        self.validate(entries)
        self.cache.reserve([(e.request_id, len(e.tokens)) for e in entries])
        logits, done, num_tokens = None, False, sum(len(e.tokens) for e in entries)
        if self.use_graphs and not (self.trace_router or self.trace_layers) and num_tokens == len(entries):
            done, logits = self._run_decode_graph(entries)
        if not done:
            ctx = self.build_context(entries)
            if self.trace_router:
                ctx.extras["router_choices"] = []
            if self.trace_layers:
                ctx.extras["layer_norms"] = []
            logits = self.model.forward(ctx)
            self.last_router_choices = ctx.extras.get("router_choices", [])
            self.last_layer_norms = ctx.extras.get("layer_norms", [])
        if self.check_kernel_status:
            self._note_status()
        for e in entries:
            self.cache.commit(e.request_id, len(e.tokens))
        self.steps_run += 1
        self.rows_run += num_tokens
        return logits

    # -- CUDA graphs for decode-only steps -------------------------------------------------------
    TABLE_WIDTH_STEP = 16      # block-table columns are rounded up to a multiple of this in a graph

    def table_width(self, request_ids) -> int:
        return max([1] + [len(self.cache.requests[r].tables[g.index]) for r in request_ids for g in self.cache.groups])

    def drop_graphs(self) -> None:
        """Forget every captured decode graph (after a failed step: a capture may have been cut short, and
        the static buffers of the others describe requests that are gone)."""
        self._graphs.clear()
        self._graph_seen.clear()
        self._graph_pool = None          # the pool goes with its last graph; the next capture makes a new one

    def reset_after_failure(self) -> None:
        """After a step that raised: no graph is trusted any more, and the kernels' status word and the
        counters they may have left behind start from zero again."""
        self.drop_graphs()
        self._status_pending = False
        if self.device.type == "cuda":
            try:
                torch.cuda.synchronize(self.device)
                ops.check_status(self.device)
            except Exception:                            # noqa: BLE001 - the failure is reported already
                pass

    def _run_decode_graph(self, entries: Sequence[StepEntry]):
        """Replay (capturing first, if this shape was seen once before) the graph of a decode-only
        step.  Returns (handled, logits); not handled means "run it eagerly this time"."""
        step = self.TABLE_WIDTH_STEP
        width = (self.table_width([e.request_id for e in entries]) + step - 1) // step * step
        # what every planner bakes into a graph (for attention: the keys of all rows together, rounded up, which
        # sizes the grid of the decode kernels whatever the longest request is)
        starts = [self.cache.requests[e.request_id].length for e in entries]
        lengths = [1] * len(entries)
        buckets = {key: p.bucket(starts, lengths) for key, p in self.planners.items()}
        key = (len(entries), sum(len(e.want) for e in entries), width, tuple(buckets.values()))
        rec = self._graphs.get(key)
        if rec is None:
            if key not in self._graph_seen:          # first sight: an eager run warms every kernel up
                self._graph_seen.add(key)
                return False, None
            rec = self._capture(entries, width, buckets)
            while len(self._graphs) >= self.max_graphs:
                self._graphs.pop(next(iter(self._graphs)))
            self._graphs[key] = rec
        else:
            rec["copied"].synchronize()              # the previous copy out of the pinned buffer is over
            self._refresh_decode(rec, entries, width, buckets)
            rec["copied"].record()
        rec["graph"].replay()
        library.launch_count += rec["launches"]     # the replay launches what the capture recorded
        self.graph_replays += 1
        self.last_router_choices = []
        return True, rec["logits"]

    def _refresh_decode(self, rec: dict, entries: Sequence[StepEntry], width: int, buckets: dict) -> None:
        """The static buffer of a captured decode step, brought up to date.  While the same requests decode
        with the same wanted places, only what moves is rewritten: token ids, positions, the block-table
        rows of requests whose tables changed (a new page, a page given back), and the planners' arrays.
        Anything else lays the whole buffer out again."""
        cache = self.cache
        ids = tuple(e.request_id for e in entries)
        wants = tuple(tuple(e.want) for e in entries)
        if rec.get("ids") != ids or rec.get("wants") != wants:
            self.build_context(entries, width=width, buffers=(rec["host"], rec["dev"]), buckets=buckets)
            rec["ids"], rec["wants"] = ids, wants
            rec["versions"] = [cache.requests[i].version for i in ids]
            return
        hv, seg, B = rec["host"].numpy(), rec["segments"], len(ids)
        starts = [cache.requests[i].length for i in ids]
        hv[seg["token_ids"][0]:seg["token_ids"][0] + B] = [e.tokens[0] for e in entries]
        hv[seg["positions"][0]:seg["positions"][0] + B] = starts       # a decode row's position is its request's length
        hv[seg["request_start"][0]:seg["request_start"][0] + B] = starts
        versions = rec["versions"]
        for b, rid in enumerate(ids):
            rc = cache.requests[rid]
            if rc.version != versions[b]:
                versions[b] = rc.version
                for g in cache.groups:
                    t = rc.tables[g.index]
                    if len(t) > width:
                        raise StepError(f"block tables need {len(t)} columns, the buffer has {width}")
                    o = seg[("table", g.index)][0] + b * width
                    hv[o:o + len(t)] = t
                    hv[o + len(t):o + width] = -1
        for key, planner in self.planners.items():
            data = planner.plan(starts, [1] * B, buckets.get(key))
            for name, arr in data.arrays.items():
                o, shape = seg[("plan", key, name)]
                arr = np.ascontiguousarray(arr, dtype=np.int32)
                if tuple(arr.shape) != shape:
                    raise StepError(f"planner {key!r}: array '{name}' changed shape inside a bucket "
                                    f"({shape} captured, {tuple(arr.shape)} now)")
                hv[o:o + arr.size] = arr.reshape(-1)
        rec["dev"].copy_(rec["host"], non_blocking=True)

    def _capture(self, entries: Sequence[StepEntry], width: int, buckets: dict) -> dict:
        hs = self.lay_out(entries, width, buckets)
        host = torch.empty(hs.words.size, dtype=torch.int32, pin_memory=True)
        dev = torch.empty(hs.words.size, dtype=torch.int32, device=self.device)
        ctx = self.build_context(entries, buffers=(host, dev), host_step=hs)
        copied = torch.cuda.Event()
        copied.record()
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        before = library.launch_count
        with torch.cuda.graph(graph, pool=self._graph_pool):
            logits = self.model.forward(ctx)
        launches = library.launch_count - before
        library.launch_count = before                # recorded, not run: replays do the counting
        if self._graph_pool is None:
            self._graph_pool = graph.pool()
        ids = tuple(e.request_id for e in entries)
        return {"graph": graph, "host": host, "dev": dev, "ctx": ctx, "logits": logits, "copied": copied,
                "launches": launches, "segments": hs.segments,
                "ids": ids, "wants": tuple(tuple(e.want) for e in entries),
                "versions": [self.cache.requests[i].version for i in ids]}
