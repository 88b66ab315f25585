#!/usr/bin/env python3
"""Where a decode step's and a prompt portion's time goes, measured on the device.

    python bench_timeline.py [--layers 4] [--batch 8] [--context 8192] [--prefill-tokens 2048] [--preset scout|maverick]

Every kernel wrapper and library product of the step is bracketed by two marker kernels that write the GPU's
nanosecond clock; the decode step is captured and replayed as in generation, so its figures contain no host
time.  A measuring tool beside ``bench.py``, not part of the package: it wraps the package's kernel wrappers
for the duration of the run.
"""
from __future__ import annotations

import argparse
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from bench import MAVERICK, SCOUT, inject_prefilled  # noqa: E402


def timeline_run(ns, cfg) -> int:
    """Where a decode step's time goes, measured inside the captured graph: every kernel wrapper and library
    product of the step is bracketed by two marker kernels that write the GPU's clock; the table gives the
    mean time between the markers per kind of call (a marker pair itself costs about 2 us, and calls on the
    second stream overlap those on the first)."""
    import collections

    import torch

    from sharpinference_b200 import Engine, EngineOptions, SamplingParams, StepEntry, build_random_model
    from sharpinference_b200.kernels import ops
    from sharpinference_b200.parts import linear as linear_mod

    dev = torch.device("cuda:0")
    B = ns.batch
    model = build_random_model(cfg, seed=0, dtype="bfloat16", device=dev, std=0.02, norm_std=0.0)
    engine = Engine(model, dtype="bfloat16", device=dev,
                    options=EngineOptions(page_size=64, max_cache_tokens=B * (ns.context + 128) + 256 + ns.prefill_tokens, max_batch=B + 1,
                                          max_tokens_per_step=max(B, 64, ns.prefill_tokens),
                                          own_dense_rows=ns.own_dense_rows))
    torch.manual_seed(0)
    for g in engine.cache.groups:
        g.kv.normal_(0.0, 1.0)
    gen = torch.Generator().manual_seed(0)
    greedy = SamplingParams(temperature=0.0, max_new_tokens=1 << 30)
    ids = [inject_prefilled(engine, torch.randint(0, cfg.vocab_size, (ns.context - 20,), generator=gen).tolist(), greedy)
           for _ in range(B)]
    reqs = [engine.request(i) for i in ids]
    slots = torch.zeros(8192, dtype=torch.int64, device=dev)
    events, state = [], {"n": 0}

    def bracket(name, fn):
        def inner(*a, **k):
            i = state["n"]
            state["n"] += 2
            ops.timestamp(slots, i)
            r = fn(*a, **k)
            ops.timestamp(slots, i + 1)
            events.append((name, i, i + 1))
            return r
        return inner

    for name in ("embed_gather", "add_rmsnorm", "swiglu", "qkv_post", "attention_decode", "router_top1",
                 "gather_rows_bf16", "tc_grouped_gemm"):
        setattr(ops, name, bracket(name, getattr(ops, name)))
    plain_call = linear_mod.Linear.__call__
    linear_mod.Linear.__call__ = lambda self, a, out=None, accumulate=False: bracket(
        f"dense product [{self.out_features} x {self.in_features}]" + (" (own kernel)" if self.streams(a) else ""),
        lambda: plain_call(self, a, out=out, accumulate=accumulate))()
    last = [r.tokens[-1] for r in reqs]
    per_step = []
    for _ in range(6):                               # the first step runs eagerly, the second is captured, then replays
        n0 = len(events)
        logits = engine.forward_step([StepEntry(i, [t], [0]) for i, t in zip(ids, last)])
        last = engine.sampler.sample(logits, [r.sampler for r in reqs])
        per_step.append(events[n0:])
    torch.cuda.synchronize()
    t = slots.cpu().tolist()
    captured = max(per_step[1:], key=len)            # the markers of the captured step hold the last replay's clocks
    table = collections.OrderedDict()
    for name, a, b in sorted(captured, key=lambda e: t[e[1]]):
        table.setdefault(name, []).append((t[b] - t[a]) / 1e3)
    first, final = min(t[a] for _, a, _ in captured), max(t[b] for _, _, b in captured)
    print(f"decode step, batch {B}, context {ns.context}, {ns.layers} layers: {(final - first) / 1e3:.1f} us from the "
          f"first marker to the last")
    for name, v in table.items():
        print(f"  {name:40s} calls {len(v):3d}   mean {sum(v) / len(v):7.1f} us   sum {sum(v):8.1f} us")

    # a prompt portion (not captured: the host launches every kernel, and is ahead of the device after the first few)
    for name in ("attention_prefill", "attention_prefill_tc"):
        setattr(ops, name, bracket(name, getattr(ops, name)))
    prompt = torch.randint(0, cfg.vocab_size, (ns.prefill_tokens,), generator=gen).tolist()
    for _ in range(3):
        n0 = len(events)
        engine.open_request("p")
        engine.forward_step([StepEntry("p", prompt, [len(prompt) - 1])])
        engine.close_request("p")
        torch.cuda.synchronize()
        last_events = events[n0:]
    t = slots.cpu().tolist()
    table = collections.OrderedDict()
    for name, a, b in sorted(last_events, key=lambda e: t[e[1]]):
        table.setdefault(name, []).append((t[b] - t[a]) / 1e3)
    first, final = min(t[a] for _, a, _ in last_events), max(t[b] for _, _, b in last_events)
    print(f"prompt portion of {ns.prefill_tokens} tokens, {ns.layers} layers: {(final - first) / 1e3:.1f} us from the first "
          f"marker to the last")
    for name, v in table.items():
        print(f"  {name:40s} calls {len(v):3d}   mean {sum(v) / len(v):7.1f} us   sum {sum(v):8.1f} us")
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--preset", default="scout", choices=["scout", "maverick"])
    ap.add_argument("--own-dense-rows", type=int, default=0,
                    help="EngineOptions.own_dense_rows: dense products of up to this many rows on the engine's own kernel")
    ns = ap.parse_args()
    from sharpinference_b200.config import Llama4TextConfig
    base = MAVERICK if ns.preset == "maverick" else SCOUT
    cfg = Llama4TextConfig.from_dict(dict(base, num_hidden_layers=ns.layers,
                                          no_rope_layers=[i for i in range(ns.layers) if (i + 1) % 4 == 0]))
    return timeline_run(ns, cfg)


if __name__ == "__main__":
    sys.exit(main())
