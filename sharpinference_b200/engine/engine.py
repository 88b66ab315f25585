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
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Union

import torch

from ..cache.manager import CacheManager
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler, SamplerState
from ..weights.loading import load_model, parse_dtype
from .scheduler import FINISHED, Request, Scheduler
from .step import StepEntry, StepRunner


@dataclass
class EngineOptions:
    """Sizes of the serving machinery.  Nothing here changes a logit."""

    page_size: int = 64                 # positions per cache page
    max_cache_tokens: Optional[int] = None   # positions every cache group can hold; None: from free memory
    memory_fraction: float = 0.85       # share of the free device memory the cache may take when sized from it
    max_batch: int = 64                 # live requests (and state slots)
    max_tokens_per_step: int = 2048     # token budget of one step
    cuda_graphs: bool = True            # capture decode-only steps as CUDA graphs (when the model's parts allow)
    # Dense bfloat16 products of steps of up to this many rows run on the engine's own tcgen05 weight-streaming
    # kernel instead of the vendor library (which the reference also uses only for batched projections, its
    # single-token products being kernels of its own).  0: the library everywhere, which measured faster on
    # B200 (Scout sizes, batch 8: 947 against 897 tok/s).  The results differ by rounding only.
    own_dense_rows: int = 0


@dataclass
class RequestOutput:
    request_id: Hashable
    prompt: List[int]
    tokens: List[int]                   # generated so far (a stop token is not included)
    finished: bool
    finish_reason: Optional[str] = None
    preemptions: int = 0


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
        self._requests: Dict[Hashable, Request] = {}
        self._ids = itertools.count()
        self.stats = {"steps": 0, "prefill_tokens": 0, "decode_tokens": 0, "preemptions": 0}

    def _size_cache(self) -> int:
        o = self.options
        if o.max_cache_tokens is not None:
            return max(1, (o.max_cache_tokens + o.page_size - 1) // o.page_size)
        per_token = 0
        itemsize = torch.empty((), dtype=self.model.act_dtype).element_size()
        for entry in self.model.schedule:
            spec = getattr(self.model.blocks[entry.layer].mixer, "cache_spec", None)
            if spec is not None and entry.cache_from is None:
                per_token += 2 * spec.num_kv_heads * spec.head_dim * itemsize
        free, _ = torch.cuda.mem_get_info(self.device)
        tokens = int(free * o.memory_fraction) // max(per_token, 1)
        tokens = max(o.page_size, min(tokens, 1 << 22))
        return tokens // o.page_size

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
        if rid in self._requests and self._requests[rid].status != FINISHED:
            raise ValueError(f"request id {rid!r} is already in use")
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

    def abort(self, request_id: Hashable) -> None:
        self.scheduler.abort(request_id)

    @property
    def has_unfinished(self) -> bool:
        return self.scheduler.has_work

    def step(self) -> List[RequestOutput]:
        """Plan one step, run it, sample, and report the requests that finished in it."""
        plan = self.scheduler.plan()
        outputs = [self._output(r) for r in plan.failed]
        self.stats["preemptions"] += len(plan.preempted)
        if not plan.entries:
            return outputs
        entries, wanting = [], []
        for e in plan.entries:
            toks = e.request.token_slice(e.start, e.count)
            entries.append(StepEntry(e.request.request_id, toks, [e.count - 1] if e.want_last else []))
            if e.want_last:
                wanting.append(e.request)
            self.stats["decode_tokens" if e.count == 1 and e.start >= len(e.request.prompt) else "prefill_tokens"] += e.count
        logits = self.runner.run(entries)
        sampled = self.sampler.sample(logits, [r.sampler for r in wanting]) if wanting else []
        if wanting:
            self.runner.flush_status()        # the sampled tokens are on the host, so the step is over: no wait
        self.stats["steps"] += 1
        for req in self.scheduler.complete(plan, sampled):
            outputs.append(self._output(req))
        return outputs

    def metrics(self) -> dict:
        """Counters of the serving machinery at this moment: what the reference's batching engine exposes as
        QueueDepth, ActiveRequests and KvTokenBudget (src/SharpInference.Engine/ContinuousBatchingEngine.cs:180-187),
        plus the pages of every cache group and the totals of ``stats``."""
        groups = {g.index: {"kind": g.spec.kind, "pages": g.pages.capacity, "free": g.pages.free_count,
                            "held": g.pages.held_count} for g in self.cache.groups}
        return {"queued": len(self.scheduler.waiting), "running": len(self.scheduler.running),
                "page_size": self.cache.page_size, "cache_groups": groups,
                "state_slots_free": self.cache.state_slots.free_count,
                "graph_replays": self.runner.graph_replays, **self.stats}

    def _output(self, req: Request) -> RequestOutput:
        return RequestOutput(req.request_id, list(req.prompt), list(req.generated), req.status == FINISHED,
                             req.finish_reason, req.preemptions)

    def output(self, request_id: Hashable) -> RequestOutput:
        return self._output(self._requests[request_id])

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
        while self.has_unfinished:
            self.step()
        self.runner.flush_status()
        outs = [self._requests[i] for i in ids]
        for r in outs:
            if r.finish_reason == "cache_full":
                raise RuntimeError(f"request {r.request_id!r} does not fit the cache "
                                   f"({self.cache.groups[0].pages.capacity} pages of {self.cache.page_size} positions)")
        return [list(r.generated) for r in outs]
