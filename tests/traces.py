"""Ways of cutting the same requests into steps, as trace records (the format ``bin/trace_run``
reads), and helpers to replay them in-process and to compare the logits with the plain
implementation."""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import torch

PAGE_ROUND = 64


def random_tokens(vocab: int, n: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def whole(requests: Dict[str, List[int]]) -> List[dict]:
    """Each request alone and whole: one step per request, every position wanted."""
    return [{"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]}
            for i, (rid, toks) in enumerate(requests.items())]


def tail_decode(requests: Dict[str, List[int]], tail: int = 32) -> List[dict]:
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps, s = [], 0
    for rid, toks in requests.items():
        head = max(len(toks) - tail, 1)
        steps.append({"step": s, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        s += 1
        for i in range(head, len(toks)):
            steps.append({"step": s, "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}],
                          "end": [rid] if i == len(toks) - 1 else []})
            s += 1
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def portions(requests: Dict[str, List[int]], sizes: Sequence[int] = (7, 2, 13, 3, 2, 5, 2, 31, 4)) -> List[dict]:
    """Portions of changing size, down to two tokens."""
    steps, s, k = [], 0, 0
    for rid, toks in requests.items():
        at = 0
        while at < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - at)
            k += 1
            steps.append({"step": s, "entries": [{"id": rid, "tokens": toks[at:at + n], "want": list(range(n))}],
                          "end": [rid] if at + n == len(toks) else []})
            at += n
            s += 1
    return steps


def mixed(requests: Dict[str, List[int]], max_live: int = 4, tail: int = 6,
          sizes: Sequence[int] = (5, 2, 9, 3, 16, 2, 7)) -> List[dict]:
    """Up to ``max_live`` requests at a time; portions of some beside single tokens of others.
    A request joins when another ends, so its pages are ones that were used before."""
    waiting = list(requests.items())
    live: List[Tuple[str, List[int], int]] = []        # id, tokens, position reached
    steps, s, k = [], 0, 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live.append((rid, toks, 0))
            if len(live) < max_live and s == 0:
                continue
            break                                        # later joiners come one per step
        entries, ended, nxt = [], [], []
        for j, (rid, toks, at) in enumerate(live):
            if (s + j) % 5 == 4 and len(live) > 1:       # now and then a request sits a step out
                nxt.append((rid, toks, at))
                continue
            left = len(toks) - at
            n = 1 if left <= tail else min(sizes[k % len(sizes)], left - tail)
            k += 1
            entries.append({"id": rid, "tokens": toks[at:at + n], "want": list(range(n))})
            if at + n == len(toks):
                ended.append(rid)
            else:
                nxt.append((rid, toks, at + n))
        live = nxt
        if entries:
            steps.append({"step": s, "entries": entries, "end": ended})
            s += 1
    return steps


def drawn(requests: Dict[str, List[int]], seed: int, max_live: int = 4,
          sizes: Sequence[int] = (1, 2, 2, 3, 5, 8, 16, 17, 31, 40), want_share: float = 0.6) -> List[dict]:
    """A drawn schedule: up to ``max_live`` requests live; each step every live request either sits out,
    brings one token, or brings a portion of a size drawn from ``sizes``; the wanted places are a drawn subset
    of the portion's places that always holds its last one."""
    import random
    r = random.Random(seed)
    waiting = list(requests.items())
    r.shuffle(waiting)
    live: List[Tuple[str, List[int], int]] = []
    steps, s = [], 0
    while waiting or live:
        while waiting and len(live) < max_live and (not live or r.random() < 0.5):
            rid, toks = waiting.pop(0)
            live.append((rid, toks, 0))
        entries, ended, nxt = [], [], []
        order = list(live)
        r.shuffle(order)
        for rid, toks, at in order:
            left = len(toks) - at
            kind = r.random()
            if kind < 0.15 and len(order) > 1:
                nxt.append((rid, toks, at))
                continue
            n = 1 if kind < 0.5 else min(left, r.choice(list(sizes)))
            want = sorted(set(i for i in range(n) if r.random() < want_share) | {n - 1})
            entries.append({"id": rid, "tokens": toks[at:at + n], "want": want})
            if at + n == len(toks):
                ended.append(rid)
            else:
                nxt.append((rid, toks, at + n))
        live = nxt
        if entries:
            steps.append({"step": s, "entries": entries, "end": ended})
            s += 1
    return steps


def max_tokens(steps: List[dict], page: int = PAGE_ROUND) -> int:
    """The most positions live requests hold at any time, each rounded up to a multiple of ``page`` (64 is
    what ``bin/trace_run`` is told; an engine with smaller pages can be given the smaller, exact figure)."""
    held: Dict[str, int] = {}
    most = 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        most = max(most, sum((n + page - 1) // page * page for n in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return most


def replay(engine, steps: List[dict], routing: Dict[str, List[List[int]]] = None
           ) -> Dict[Tuple[str, int], torch.Tensor]:
    """Run the steps through the engine below its scheduler, as trace_run does; logits (CPU,
    float32) by (request id, position).  If ``routing`` is a dict it receives, per request, the
    expert every token was sent to in every routed layer: ``routing[id][routed layer][position]``."""
    from sharpinference_b200 import StepEntry
    out: Dict[Tuple[str, int], torch.Tensor] = {}
    at: Dict[str, int] = {}
    engine.runner.trace_router = routing is not None
    for st in steps:
        entries = []
        for e in st["entries"]:
            if e["id"] not in at:
                engine.open_request(e["id"])
                at[e["id"]] = 0
            entries.append(StepEntry(e["id"], e["tokens"], e["want"]))
        logits = engine.forward_step(entries)
        rows = logits.float().cpu() if logits is not None else None
        if routing is not None:
            picks = [c.cpu().tolist() for c in engine.runner.last_router_choices]
            row = 0
            for e in st["entries"]:
                per_layer = routing.setdefault(e["id"], [[] for _ in picks])
                for layer, p in enumerate(picks):
                    per_layer[layer].extend(p[row:row + len(e["tokens"])])
                row += len(e["tokens"])
        r = 0
        for e in st["entries"]:
            for wpos in e["want"]:
                out[(e["id"], at[e["id"]] + wpos)] = rows[r]
                r += 1
            at[e["id"]] += len(e["tokens"])
        for rid in st["end"]:
            engine.close_request(rid)
            del at[rid]
    return out


def worst_error(got: Dict[Tuple[str, int], torch.Tensor], expected: Dict[str, torch.Tensor]):
    """Largest |difference| over all wanted rows, relative to the largest |logit| of the
    request's expected logits; also where it is.  Returns (error, (request, position))."""
    worst, where = 0.0, None
    for (rid, pos), row in got.items():
        ref = expected[rid]
        scale = float(ref.abs().max())
        err = float((row.double() - ref[pos].double()).abs().max()) / scale
        if not err <= worst:          # also catches NaN
            worst, where = err, (rid, pos)
    return worst, where
