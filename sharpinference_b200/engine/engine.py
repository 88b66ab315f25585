"""``Engine``: the Python entry point.  Model + cache manager + step function + scheduler + sampler.

The reference's programming interface is ``IInferenceEngine.GenerateChunksAsync(prompt,
SamplingParams, ct)`` over a forward pass and a tokenizer
(src/SharpInference.Engine/IInferenceEngine.cs:61-65, samples/SharpInference.Sample.Chat/Program.cs);
its batched engine adds requests to a queue that one loop serves
(src/SharpInference.Engine/ContinuousBatchingEngine.cs:224-255).  Here prompts are token ids
(random-weight models have no vocabulary) and the loop is driven by the caller:

    eng = Engine("model_dir", dtype="bfloat16")
    outs = eng.generate([[1, 2, 3], [4, 5]], SamplingParams(temperature=0, max_new_tokens=8))

or request by request: ``add_request`` / ``step`` / ``has_unfinished``; or below the scheduler:
``open_request`` / ``forward_step`` / ``close_request``, which is what trace replay uses.
"""
from __future__ import annotations

import itertools
from collections import OrderedDict
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Union

import torch

from ..cache.manager import CacheManager, OutOfPages
from ..cache.sizing import group_layout, pages_per_group
from ..kernels import library
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler, SamplerState
from ..weights.loading import load_model, parse_dtype
from .scheduler import FINISHED, Request, Scheduler, StepPlan
from .step import StepEntry, StepError, StepRunner


@dataclass
class EngineOptions:
    """Sizes of the serving machinery.  Nothing here changes a logit."""

    page_size: int = 64                 # positions per cache page
    # positions every cache group can hold; None: from free memory, each group by its needs (a group whose mask
    # forgets the past is sized for max_batch requests of its span plus a step, the rest goes to the others)
    max_cache_tokens: Optional[int] = None
    memory_fraction: float = 0.85       # share of the free device memory the cache may take when sized from it
    max_batch: int = 64                 # live requests (and state slots)
    max_tokens_per_step: int = 2048     # token budget of one step
    cuda_graphs: bool = True            # capture decode-only steps as CUDA graphs (when the model's parts allow)
    # Dense bfloat16 products of steps of up to this many rows (at most 16) run on the engine's own
    # weight-streaming kernel instead of the vendor library (which the reference also uses only for batched
    # projections, its single-token products being kernels of its own).  0: the library everywhere, which is
    # the faster step on B200 (Scout sizes, 8 layers, batch 1: 614 against 593 tok/s) although the own kernel
    # is the faster product alone (parts/linear.py has the figures).  The LM head keeps the library either way
    # (2 GB of weights: 322 against 299 us).  The results differ by rounding only.
    own_dense_rows: int = 0
    # Launch kernels with programmatic stream serialization: a kernel's set-up overlaps the tail of the one
    # before it.  False launches every kernel the plain way.  One switch for the process (the kernel libraries
    # are shared by every engine in it).
    programmatic_launch: bool = True
    keep_finished: int = 1024           # finished requests whose output `output()` can still give


@dataclass
class RequestOutput:
    request_id: Hashable
    prompt: List[int]
    tokens: List[int]                   # generated so far (a stop token is not included)
    finished: bool
    finish_reason: Optional[str] = None     # stop, length, abort, cache_full, error
    preemptions: int = 0
    error: Optional[str] = None             # the message, when finish_reason is "error"


def _linears(root, depth: int = 4, seen=None):
    """Every :class:`Linear` reachable from a model through attributes, lists and tuples."""
    from ..parts.linear import Linear
    seen = set() if seen is None else seen
    if id(root) in seen or depth < 0:
        return
    seen.add(id(root))
    if isinstance(root, Linear):
        yield root
        return
    if isinstance(root, (list, tuple)):
        for item in root:
            yield from _linears(item, depth, seen)
        return
    if isinstance(root, torch.Tensor) or not hasattr(root, "__dict__"):
        return
    for value in vars(root).values():
        yield from _linears(value, depth - 1, seen)


class Engine:
    def __init__(self, model: Union[str, object], *, dtype="bfloat16", device="cuda:0",
                 options: Optional[EngineOptions] = None):
        self.device = torch.device(device)
        if self.device.type != "cuda" or not torch.cuda.is_available():
            raise RuntimeError("the engine runs on a CUDA device only (its kernels are compiled for sm_100a); "
                               f"device {device!r} with torch.cuda.is_available()={torch.cuda.is_available()}")
        self.options = options or EngineOptions()
        self.dtype = parse_dtype(dtype)
        torch.cuda.set_device(self.device)
        self.model = load_model(model, self.dtype, self.device) if isinstance(model, str) else model
        o = self.options
        library.set_programmatic_launch(o.programmatic_launch)
        if o.own_dense_rows > 0:
            for lin in _linears(self.model):
                if lin is not getattr(self.model, "head", None):      # the LM head streams 2 GB: the library's job
                    lin.stream_rows = o.own_dense_rows
        num_pages = self._size_cache()
        self.cache = CacheManager(self.model.schedule, self.model.blocks, page_size=o.page_size,
                                  num_pages=num_pages, max_requests=o.max_batch, dtype=self.model.act_dtype,
                                  device=self.device)
        self.runner = StepRunner(self.model, self.cache)
        self.runner.use_graphs = self.runner.use_graphs and o.cuda_graphs
        self.scheduler = Scheduler(self.cache, max_batch=o.max_batch, max_tokens_per_step=o.max_tokens_per_step)
        self.sampler = Sampler(self.device)
        self._start_bookkeeping()

    @classmethod
    def from_parts(cls, *, model, cache, runner, sampler, options: Optional[EngineOptions] = None) -> "Engine":
        """An engine around a given model, cache manager, step function and sampler (any object with ``run``,
        ``flush_status`` and ``reset_after_failure``, and with ``sample``): how tests drive the request loop
        with stand-ins, without a device."""
        self = cls.__new__(cls)
        self.options = options or EngineOptions()
        self.device, self.dtype = getattr(cache, "device", None), getattr(model, "act_dtype", None)
        self.model, self.cache, self.runner, self.sampler = model, cache, runner, sampler
        self.scheduler = Scheduler(cache, max_batch=self.options.max_batch,
                                   max_tokens_per_step=self.options.max_tokens_per_step)
        self._start_bookkeeping()
        return self

    def _start_bookkeeping(self) -> None:
        self._requests: Dict[Hashable, Request] = {}                # waiting and running
        self._finished: "OrderedDict[Hashable, Request]" = OrderedDict()   # the last `keep_finished` that ended
        self._ids = itertools.count()
        self.stats = {"steps": 0, "prefill_tokens": 0, "decode_tokens": 0, "preemptions": 0, "failed_steps": 0}
        self.last_error: Optional[BaseException] = None

    def _size_cache(self):
        """Pages per cache group: one number for all when ``max_cache_tokens`` says so, else from the free
        device memory, each group by its needs."""
        o = self.options
        if o.max_cache_tokens is not None:
            return max(1, (o.max_cache_tokens + o.page_size - 1) // o.page_size)
        groups = group_layout(self.model.schedule, self.model.blocks)
        itemsize = torch.empty((), dtype=self.model.act_dtype).element_size()
        free, _ = torch.cuda.mem_get_info(self.device)
        pages = pages_per_group(groups, budget_bytes=int(free * o.memory_fraction), itemsize=itemsize,
                                page_size=o.page_size, max_batch=o.max_batch,
                                max_tokens_per_step=o.max_tokens_per_step)
        return dict(enumerate(pages)) if pages else 1

    # -- below the scheduler ---------------------------------------------------------------
    def open_request(self, request_id: Hashable) -> None:
        self.cache.add_request(request_id)

    def close_request(self, request_id: Hashable) -> None:
        self.cache.free_request(request_id)

    def forward_step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """One step of the step function: float32 logits [wanted, vocab] on the device."""
        return self.runner.run(entries)

    # -- requests ----------------------------------------------------------------------------
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None,
                    request_id: Optional[Hashable] = None) -> Hashable:
        params = params or SamplingParams()
        rid = request_id if request_id is not None else next(self._ids)
        if rid in self._requests:
            raise ValueError(f"request id {rid!r} is already in use")
        self._finished.pop(rid, None)
        prompt = [int(t) for t in prompt]
        V = self.model.vocab_size
        for t in prompt:
            if not (0 <= t < V):
                raise ValueError(f"prompt token {t} is outside the vocabulary [0, {V})")
        req = Request(rid, prompt, params, stop_set=params.resolve_stop_set(self.model.eos_token_ids),
                      sampler=SamplerState.start(params, prompt))
        self.scheduler.add(req)
        self._requests[rid] = req
        return rid

    def abort(self, request_id: Hashable) -> Optional[RequestOutput]:
        req = self.scheduler.abort(request_id)
        return self._report(req) if req is not None else None

    @property
    def has_unfinished(self) -> bool:
        return self.scheduler.has_work

    def step(self) -> List[RequestOutput]:
        """Plan one step, run it, sample, and report the requests that ended in it.

        A step that cannot run does not take the engine down with it
        (src/SharpInference.Engine/ContinuousBatchingEngine.cs:465-501, :529-535, :662-672):

        * one request cannot run as given (a token outside the vocabulary, ...): it is found before anything
          is reserved or launched; that request ends with ``finish_reason="error"`` and the step is planned
          again without it;
        * the cache has fewer pages than the plan counted on: nothing was taken; the scheduler's out-of-pages
          rule is applied (the newest running request goes back to the queue) and the step is planned again;
        * anything else (a kernel that gave up on a wait, a failed launch, an exception in a part or in the
          sampler) leaves the caches of the step in an unknown state: every running and waiting request ends
          with ``finish_reason="error"`` and the message, their pages and state slots are given back, captured
          graphs are dropped, the exception is kept in ``last_error``, and the engine takes new requests.
        """
        outputs: List[RequestOutput] = []
        for _ in range(2 * self.options.max_batch + 4):      # every retry ends or sends back a request
            plan = self.scheduler.plan()
            outputs.extend(self._report(r) for r in plan.failed)
            self.stats["preemptions"] += len(plan.preempted)
            if not plan.entries:
                return outputs
            try:
                outputs.extend(self._run_plan(plan))
                return outputs
            except StepError as exc:
                req = self._requests.get(exc.request_id)
                if req is None:
                    outputs.extend(self._fail_everything(exc))
                    return outputs
                self.scheduler.fail(req, str(exc))
                outputs.append(self._report(req))
            except OutOfPages:
                retry = StepPlan()
                self.scheduler.preempt_newest(retry)
                self.stats["preemptions"] += len(retry.preempted)
                outputs.extend(self._report(r) for r in retry.failed)
            except Exception as exc:                     # noqa: BLE001 - the loop must outlive any failed step
                outputs.extend(self._fail_everything(exc))
                return outputs
        outputs.extend(self._fail_everything(RuntimeError("the step could not be planned after repeated failures")))
        return outputs

    def _run_plan(self, plan: StepPlan) -> List[RequestOutput]:
        entries, wanting = [], []
        prefill = decode = 0
        for e in plan.entries:
            toks = e.request.token_slice(e.start, e.count)
            entries.append(StepEntry(e.request.request_id, toks, [e.count - 1] if e.want_last else []))
            if e.want_last:
                wanting.append(e.request)
            if e.count == 1 and e.start >= len(e.request.prompt):
                decode += 1
            else:
                prefill += e.count
        logits = self.runner.run(entries)
        sampled = self.sampler.sample(logits, [r.sampler for r in wanting]) if wanting else []
        if wanting:
            self.runner.flush_status()        # the sampled tokens are on the host, so the step is over: no wait
        self.stats["steps"] += 1
        self.stats["prefill_tokens"] += prefill
        self.stats["decode_tokens"] += decode
        return [self._report(req) for req in self.scheduler.complete(plan, sampled)]

    def _fail_everything(self, exc: BaseException) -> List[RequestOutput]:
        self.last_error = exc
        self.stats["failed_steps"] += 1
        failed = self.scheduler.fail_all(f"{type(exc).__name__}: {exc}")
        self.runner.reset_after_failure()
        return [self._report(r) for r in failed]

    def _report(self, req: Request) -> RequestOutput:
        """The output of a request; one that has ended moves from the live table to the bounded history."""
        if req.status == FINISHED and self._requests.pop(req.request_id, None) is not None:
            self._finished[req.request_id] = req
            while len(self._finished) > max(self.options.keep_finished, 0):
                self._finished.popitem(last=False)
        return self._output(req)

    def metrics(self) -> dict:
        """Counters of the serving machinery at this moment: what the reference's batching engine exposes as
        QueueDepth, ActiveRequests and KvTokenBudget (src/SharpInference.Engine/ContinuousBatchingEngine.cs:180-187),
        plus the pages of every cache group and the totals of ``stats``."""
        groups = {g.index: {"kind": g.spec.kind, "pages": g.pages.capacity, "free": g.pages.free_count,
                            "held": g.pages.held_count} for g in self.cache.groups}
        return {"queued": len(self.scheduler.waiting), "running": len(self.scheduler.running),
                "tracked_requests": len(self._requests),
                "page_size": self.cache.page_size, "cache_groups": groups,
                "state_slots_free": self.cache.state_slots.free_count,
                "graph_replays": getattr(self.runner, "graph_replays", 0), **self.stats}

    def _output(self, req: Request) -> RequestOutput:
        return RequestOutput(req.request_id, list(req.prompt), list(req.generated), req.status == FINISHED,
                             req.finish_reason, req.preemptions, req.error)

    def request(self, request_id: Hashable) -> Request:
        """The scheduler's record of a live request, or of one of the last ``keep_finished`` that ended."""
        req = self._requests.get(request_id)
        if req is None:
            req = self._finished.get(request_id)
        if req is None:
            raise KeyError(f"request {request_id!r} is neither live nor among the last "
                           f"{self.options.keep_finished} that ended")
        return req

    def output(self, request_id: Hashable) -> RequestOutput:
        return self._output(self.request(request_id))

    def generate(self, prompts: Sequence[Sequence[int]],
                 params: Union[SamplingParams, Sequence[SamplingParams], None] = None) -> List[List[int]]:
        """Generate for every prompt (token ids in, token ids out), batched continuously."""
        if params is None or isinstance(params, SamplingParams):
            plist = [params or SamplingParams()] * len(prompts)
        else:
            plist = list(params)
            if len(plist) != len(prompts):
                raise ValueError(f"{len(prompts)} prompts but {len(plist)} sampling parameter sets")
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, plist)]
        done: Dict[Hashable, RequestOutput] = {}
        while self.has_unfinished:
            for out in self.step():
                done[out.request_id] = out
        try:
            self.runner.flush_status()
        except Exception as exc:                         # noqa: BLE001 - a kernel of the last step gave up
            self._fail_everything(exc)
            raise
        outs = [done[i] if i in done else self.output(i) for i in ids]
        for r in outs:
            if r.finish_reason == "cache_full":
                raise RuntimeError(f"request {r.request_id!r} does not fit the cache "
                                   f"({self.cache.groups[0].pages.capacity} pages of {self.cache.page_size} positions)")
            if r.finish_reason == "error":
                raise RuntimeError(f"request {r.request_id!r} failed: {r.error}") from self.last_error
        return [list(r.tokens) for r in outs]
