#!/usr/bin/env python3
"""Throughput of the engine on one B200: decoded tokens per second at a batch and context, plus
prefill, a roofline figure for the decode step and two further batch sizes.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch B] [--context S]

One JSON line on standard output.  The default run has the layer sizes of Llama-4-Scout with
random bfloat16 weights (20 layers), batch 8, context 8192.  ``value`` is decoded tokens per
second of the step function plus sampling, timed with CUDA events; ``e2e`` is the same through
``Engine.step()`` with token ids going in from (pinned) host memory and sampled ids coming back to
the host every step.  ``--impl reference`` reports that the reference cannot run here.  Beside this file:
``bench_timeline.py`` (where a step's time goes, from clock markers inside the replayed graph) and
``bench_kernels.py`` (one kernel at model sizes).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SCOUT = dict(
    vocab_size=202048, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, head_dim=128,
    intermediate_size=8192, intermediate_size_mlp=16384, num_local_experts=16, num_experts_per_tok=1,
    interleave_moe_layer_step=1, rope_theta=500000.0,
    rope_scaling={"rope_type": "llama3", "factor": 16.0, "low_freq_factor": 1.0, "high_freq_factor": 1.0,
                  "original_max_position_embeddings": 8192},
    attention_chunk_size=8192, use_qk_norm=True, attn_temperature_tuning=True, floor_scale=8192, attn_scale=0.1,
    rms_norm_eps=1e-5, tie_word_embeddings=False,
)
SCOUT_FULL_LAYERS = 48
# Llama-4-Maverick layer sizes: dense SwiGLU (16384) and 128-expert layers alternate.
MAVERICK = dict(SCOUT, num_local_experts=128, interleave_moe_layer_step=2, intermediate_size_mlp=16384,
                rope_scaling=None)
MAVERICK_FULL_LAYERS = 48
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as fh:
                got = json.load(fh)
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if isinstance(got.get(k), (int, float)) and got[k] > 0:
                    out[k] = float(got[k])
            return out, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi sampling SM clocks and throttle reasons while a region is timed."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.path = tempfile.mktemp(prefix="clocks_", suffix=".csv")
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            with open(self.path) as fh:
                for line in fh:
                    parts = [p.strip() for p in line.split(",")]
                    if len(parts) < 7:
                        continue
                    try:
                        sm.append(float(parts[0]))
                        mx.append(float(parts[1]))
                    except ValueError:
                        continue
                    for name, val in zip(names, parts[3:7]):
                        if val.lower().startswith("active"):
                            reasons.add(name)
            os.remove(self.path)
        except OSError:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def layer_counts(cfg):
    nope = [i for i in range(cfg.num_hidden_layers) if not cfg.layer_uses_rope(i)]
    return cfg.num_hidden_layers - len(nope), len(nope)


def decode_bytes(cfg, batch, context, distinct_experts_per_layer, itemsize=2):
    """Bytes a decode step has to read: every weight it uses once, and the cache of the live requests.
    ``distinct_experts_per_layer`` has one entry per mixture layer, in layer order."""
    H, d, nq, nkv, I = cfg.hidden_size, cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.intermediate_size
    attention = ((nq + 2 * nkv) * d * H + H * nq * d) * itemsize + 2 * H * 4
    mixture = 3 * H * I * itemsize + cfg.num_local_experts * H * 4                  # shared expert and router
    dense = 3 * H * cfg.intermediate_size_mlp * itemsize
    moe_layers = sum(cfg.layer_is_moe(i) for i in range(cfg.num_hidden_layers))
    weights = cfg.num_hidden_layers * attention + moe_layers * mixture + (cfg.num_hidden_layers - moe_layers) * dense
    weights += sum(distinct_experts_per_layer) * 3 * H * I * itemsize
    weights += cfg.vocab_size * H * itemsize + batch * H * itemsize + H * 4
    rope_layers, nope_layers = layer_counts(cfg)
    pos = context - 1
    chunk_keys = pos - (pos // cfg.attention_chunk_size) * cfg.attention_chunk_size + 1
    cache = batch * 2 * nkv * d * itemsize * (rope_layers * chunk_keys + nope_layers * (pos + 1))
    return weights + cache


def prefill_flops(cfg, tokens, start=0):
    """Flops of a prompt portion of ``tokens`` rows whose first row is at position ``start`` (logits at one row)."""
    H, d, nq, nkv, I, V = (cfg.hidden_size, cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads,
                           cfg.intermediate_size, cfg.vocab_size)
    attention = 2 * H * (nq + 2 * nkv) * d + 2 * H * nq * d
    mixture = 2 * H * cfg.num_local_experts + 2 * 2 * 3 * H * I          # router, shared and routed expert
    dense = 2 * 3 * H * cfg.intermediate_size_mlp
    moe_layers = sum(cfg.layer_is_moe(i) for i in range(cfg.num_hidden_layers))
    per_token = cfg.num_hidden_layers * attention + moe_layers * mixture + (cfg.num_hidden_layers - moe_layers) * dense
    # (query, key) pairs: a global layer's query at position p sees p + 1 keys, a chunked layer's p % chunk + 1
    C = cfg.attention_chunk_size
    full_pairs = sum(p + 1 for p in range(start, start + tokens))
    chunk_pairs = sum(p % C + 1 for p in range(start, start + tokens))
    rope_layers, nope_layers = layer_counts(cfg)
    attn = 4 * nq * d * (rope_layers * chunk_pairs + nope_layers * full_pairs)
    return tokens * per_token + attn + 2 * V * H


def prefill_floor_ms(cfg, tokens, pk, start=0):
    """The least time a prompt step can take at the peaks given: the routed experts' products at the slower
    of their flops and the bytes of the experts touched (at most one per token), everything else at its
    flops.  With 16 experts and 2048 tokens the routed products are bound by memory."""
    H, I = cfg.hidden_size, cfg.intermediate_size
    routed_flops = tokens * 2 * 3 * H * I
    routed_bytes = min(cfg.num_local_experts, tokens) * 3 * H * I * 2
    flops_s, bytes_s = pk["bf16_tflops"] * 1e12, pk["hbm_gbs"] * 1e9
    routed = max(routed_flops / flops_s, routed_bytes / bytes_s)
    moe_layers = sum(cfg.layer_is_moe(i) for i in range(cfg.num_hidden_layers))
    rest = (prefill_flops(cfg, tokens, start) - moe_layers * routed_flops) / flops_s
    return (moe_layers * routed + rest) * 1e3


def inject_prefilled(engine, prompt, params):
    """Benchmark glue: a running request whose first len(prompt) - 1 positions are already cached
    (the pool holds random keys and values), so the next step decodes at that context."""
    from sharpinference_b200.engine.scheduler import RUNNING
    rid = engine.add_request(prompt, params)
    req = engine.scheduler.waiting.pop()
    assert req.request_id == rid
    engine.cache.add_request(rid)
    n = len(prompt) - 1
    engine.cache.reserve([(rid, n)])
    engine.cache.commit(rid, n)
    req.computed, req.status = n, RUNNING
    engine.scheduler.running.append(req)
    return rid


def long_context_run(ns, cfg, pk, pk_kind) -> int:
    """One request with a 65536-token prompt, prefilled through the engine in 2048-token portions, then
    256 decoded tokens.  The prompt crosses eight attention chunks: the chunked layers give their pages
    back behind the live chunk, the global layers keep the whole history."""
    import torch

    from sharpinference_b200 import Engine, EngineOptions, SamplingParams, build_random_model

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    prompt_len, portion, new_tokens, page = 65536, ns.prefill_tokens, 256, 64
    model = build_random_model(cfg, seed=0, dtype="bfloat16", device=dev, std=0.02, norm_std=0.0)
    engine = Engine(model, dtype="bfloat16", device=dev,
                    options=EngineOptions(page_size=page, max_cache_tokens=prompt_len + new_tokens + 2 * page, max_batch=1,
                                          max_tokens_per_step=portion))
    gen = torch.Generator().manual_seed(0)
    # untimed: a short request first, so that kernels are loaded, the library has chosen its routines and the
    # allocator holds its blocks when the clock starts
    warm = torch.randint(0, cfg.vocab_size, (2 * portion + 5,), generator=gen).tolist()
    engine.generate([warm], SamplingParams(temperature=0.0, max_new_tokens=4))
    prompt = torch.randint(0, cfg.vocab_size, (prompt_len,), generator=gen).tolist()
    rid = engine.add_request(prompt, SamplingParams(temperature=0.0, max_new_tokens=new_tokens))
    req = engine.request(rid)
    chunk_group = [g for g in engine.cache.groups if g.spec.kind == "chunk"][0].index
    full_group = [g for g in engine.cache.groups if g.spec.kind == "full"][0].index
    most_chunk_pages = 0
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    portions = 0
    while not req.generated:
        engine.step()
        portions += 1
        most_chunk_pages = max(most_chunk_pages, engine.cache.held_pages(rid)[chunk_group])
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    full_pages = engine.cache.held_pages(rid)[full_group]
    settle = 32                      # decode steps before the clock starts: the step's graph is captured in them
    for _ in range(settle):
        engine.step()
    torch.cuda.synchronize()
    t1d = time.perf_counter()
    while engine.has_unfinished:
        engine.step()
    torch.cuda.synchronize()
    t2 = time.perf_counter()
    timed_tokens = new_tokens - 1 - settle
    dec_ms = (t2 - t1d) * 1e3 / timed_tokens
    # the decode step's roofline: every weight it uses once (one expert a layer) and the request's cache at the
    # middle of the timed stretch
    mid_context = prompt_len + settle + timed_tokens // 2
    moe_layers = sum(cfg.layer_is_moe(i) for i in range(cfg.num_hidden_layers))
    need = decode_bytes(cfg, 1, mid_context, [1.0] * moe_layers)
    achieved = need / (dec_ms * 1e-3) / 1e9
    floor_ms = sum(prefill_floor_ms(cfg, portion, pk, start) for start in range(0, prompt_len, portion))
    flops = sum(prefill_flops(cfg, portion, start) for start in range(0, prompt_len, portion))
    out = {
        "metric": "long context: prefill tok/s over a 65536-token prompt in 2048-token portions, then decode tok/s",
        "impl": "ours", "n_gpus": 1, "dtype": "bf16", "data": "synthetic: random weights, uniform random token ids",
        "prefill": {"value": prompt_len / (t1 - t0), "unit": "tokens/s", "tokens": prompt_len, "portions": portions,
                    "ms": (t1 - t0) * 1e3, "frac": flops / (t1 - t0) / (pk["bf16_tflops_sustained"] * 1e12),
                    "peak_tflops": pk["bf16_tflops_sustained"], "peak": pk_kind + ", sustained (a seconds-long run)",
                    "floor_ms": floor_ms, "frac_of_floor": floor_ms / ((t1 - t0) * 1e3)},
        "decode": {"value": timed_tokens / (t2 - t1d), "unit": "tokens/s", "tokens": timed_tokens,
                   "ms_per_step": dec_ms},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "bytes_per_step": need, "peak_kind": pk_kind,
                     "context": mid_context},
        "cache": {"page_size": page, "chunk_group_pages_at_most": most_chunk_pages,
                  "chunk_group_positions_at_most": most_chunk_pages * page,
                  "global_group_pages_after_prefill": full_pages},
        "config": {"model": "llama4-scout-sizes", "layers": ns.layers, "layers_full_model": SCOUT_FULL_LAYERS,
                   "hidden": cfg.hidden_size, "q_heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "experts": cfg.num_local_experts, "chunk": cfg.attention_chunk_size,
                   "prompt": prompt_len, "portion": portion, "new_tokens": new_tokens},
    }
    print(json.dumps(out))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=20)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--own-dense-rows", type=int, default=0,
                    help="EngineOptions.own_dense_rows: dense products of up to this many rows on the engine's own kernel")
    ap.add_argument("--points", default="1,64", help="further decode batch sizes, comma separated ('' for none)")
    ap.add_argument("--preset", default="scout", choices=["scout", "maverick", "long"],
                    help="scout: 20 Scout-sized layers, batch 8 at context 8192 (the default run); maverick: 4 "
                         "Maverick-sized layers (dense / 128 experts alternating), batch 64 at context 4096; long: 8 "
                         "Scout-sized layers, one 65536-token prompt prefilled in 2048-token portions, then 256 "
                         "decoded tokens")
    ns = ap.parse_args()
    if ns.preset == "maverick":
        defaults = ap.parse_args([])
        ns.layers = 4 if ns.layers == defaults.layers else ns.layers
        ns.batch = 64 if ns.batch == defaults.batch else ns.batch
        ns.context = 4096 if ns.context == defaults.context else ns.context
        ns.points = "" if ns.points == defaults.points else ns.points
    if ns.preset == "long":
        ns.layers = 8 if ns.layers == ap.get_default("layers") else ns.layers

    if ns.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "pekkah/SharpInference is C#/.NET 10 with no Python package metadata; pip cannot install "
                          "it offline and no .NET runtime is on this machine"}))
        return 0
    if ns.gpus != 1:
        print(f"bench.py measures one GPU: this engine is single-GPU by design (asked for --gpus {ns.gpus})")
        return 2
    warmup, steps = max(ns.warmup, 3), max(ns.steps, 1)

    import torch

    from sharpinference_b200 import Engine, EngineOptions, SamplingParams, StepEntry, build_random_model
    from sharpinference_b200.config import Llama4TextConfig
    from sharpinference_b200.kernels import library

    base = MAVERICK if ns.preset == "maverick" else SCOUT
    cfg = Llama4TextConfig.from_dict(dict(base, num_hidden_layers=ns.layers,
                                          no_rope_layers=[i for i in range(ns.layers) if (i + 1) % 4 == 0]))
    pk, pk_kind = peaks()
    if ns.preset == "long":
        return long_context_run(ns, cfg, pk, pk_kind)
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    t0 = time.time()
    model = build_random_model(cfg, seed=0, dtype="bfloat16", device=dev, std=0.02, norm_std=0.0)
    torch.cuda.synchronize()
    batches = [ns.batch] + [int(b) for b in ns.points.split(",") if b.strip()]
    max_b = max(batches)
    page = 64
    cache_tokens = max_b * ((ns.context + page - 1) // page * page + page) + ns.prefill_tokens + page
    engine = Engine(model, dtype="bfloat16", device=dev,
                    options=EngineOptions(page_size=page, max_cache_tokens=cache_tokens, max_batch=max_b,
                                          max_tokens_per_step=max(ns.prefill_tokens, max_b),
                                          own_dense_rows=ns.own_dense_rows))
    torch.manual_seed(0)                   # the cache content decides the routing of the timed steps: keep it fixed
    for g in engine.cache.groups:          # keys and values as a prefill would have left them: unit-scale numbers
        g.kv.normal_(0.0, 1.0)
    print(f"[bench] model and cache ready in {time.time() - t0:.1f} s, "
          f"{torch.cuda.memory_allocated() / 2**30:.1f} GiB allocated", file=sys.stderr, flush=True)
    gen = torch.Generator().manual_seed(0)

    def tokens(n):
        return torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist()

    greedy = SamplingParams(temperature=0.0, max_new_tokens=1 << 30)

    # ---- prefill of one prompt from an empty cache ---------------------------------------
    prompt = tokens(ns.prefill_tokens)
    pre_ms = []
    for it in range(warmup + 3):
        engine.open_request("p")
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        engine.forward_step([StepEntry("p", prompt, [len(prompt) - 1])])
        b.record()
        torch.cuda.synchronize()
        engine.close_request("p")
        if it >= warmup:
            pre_ms.append(a.elapsed_time(b))
    pre = statistics.median(pre_ms)
    prefill = {"value": ns.prefill_tokens / pre * 1e3, "tokens": ns.prefill_tokens, "ms": pre,
               "frac": prefill_flops(cfg, ns.prefill_tokens) / (pre * 1e-3) / (pk["bf16_tflops"] * 1e12),
               "peak_tflops": pk["bf16_tflops"], "peak": pk_kind,
               # beside the contract's flops fraction: against the step's own floor, whose routed experts are
               # bound by the bytes of their weights
               "floor_ms": prefill_floor_ms(cfg, ns.prefill_tokens, pk)}
    prefill["frac_of_floor"] = prefill["floor_ms"] / pre

    # ---- decode -----------------------------------------------------------------------------
    def decode_run(B, timed_steps, through_engine):
        """B requests at `context`; returns (ms per step, distinct experts per layer, bytes moved per step)."""
        traced = 0 if through_engine else 4           # eager steps that record which experts the batch uses
        total = warmup + timed_steps + traced
        ids = [inject_prefilled(engine, tokens(ns.context - total), greedy) for _ in range(B)]
        reqs = [engine.request(i) for i in ids]
        h2d = d2h = 0
        distinct = None
        launches0 = 0
        if through_engine:
            for _ in range(warmup):
                engine.step()
            torch.cuda.synchronize()
            launches0 = library.launch_count
            t_start = time.perf_counter()
            for _ in range(timed_steps):
                engine.step()
            torch.cuda.synchronize()
            ms = (time.perf_counter() - t_start) * 1e3 / timed_steps
            width = max(len(engine.cache.requests[i].tables[g.index]) for i in ids for g in engine.cache.groups)
            h2d = 4 * (3 * B + B + (B + 1) + B + B + len(engine.cache.groups) * B * width)
            d2h = 4 * B
        else:
            last = [r.tokens[-1] for r in reqs]
            engine.runner.trace_router = True        # distinct experts per mixture layer, the mean of a few steps
            counts = []
            for _ in range(traced):
                logits = engine.forward_step([StepEntry(i, [t], [0]) for i, t in zip(ids, last)])
                last = engine.sampler.sample(logits, [r.sampler for r in reqs])
                counts.append([len(set(c.tolist())) for c in engine.runner.last_router_choices])
            distinct = [round(sum(col) / traced, 2) for col in zip(*counts)]
            engine.runner.trace_router = False
            for _ in range(warmup):                   # includes the capture of this shape's CUDA graph
                logits = engine.forward_step([StepEntry(i, [t], [0]) for i, t in zip(ids, last)])
                last = engine.sampler.sample(logits, [r.sampler for r in reqs])
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            launches0 = library.launch_count
            a.record()
            for _ in range(timed_steps):
                logits = engine.forward_step([StepEntry(i, [t], [0]) for i, t in zip(ids, last)])
                last = engine.sampler.sample(logits, [r.sampler for r in reqs])
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b) / timed_steps
        launches = library.launch_count - launches0
        for i in ids:
            engine.abort(i)
        return ms, distinct, h2d, d2h, launches

    with ClockSampler() as clocks:
        ms, distinct, _, _, launches = decode_run(ns.batch, steps, through_engine=False)
    clock_summary = clocks.summary()
    e2e_ms, _, h2d, d2h, _ = decode_run(ns.batch, steps, through_engine=True)
    e2e_b1_ms = decode_run(1, max(3, steps // 2), through_engine=True)[0] if 1 in batches[1:] else None
    need = decode_bytes(cfg, ns.batch, ns.context, distinct)
    achieved = need / (ms * 1e-3) / 1e9
    points = {}
    for b in batches[1:]:
        pms, pdistinct, _, _, _ = decode_run(b, max(3, steps // 2), through_engine=False)
        points[f"decode_b{b}"] = b / pms * 1e3
        # the same roofline figure as for the headline batch: bytes the step has to read / its time / the peak
        points[f"decode_b{b}_roofline_frac"] = decode_bytes(cfg, b, ns.context, pdistinct) / (pms * 1e-3) / 1e9 / pk["hbm_gbs"]
    if e2e_b1_ms is not None:           # what the host adds at batch 1: the same steps through Engine.step()
        points["decode_b1_e2e"] = 1 / e2e_b1_ms * 1e3

    out = {
        "metric": f"decode tok/s @ batch {ns.batch}, context {ns.context} "
                  f"(Llama-4-{'Maverick' if ns.preset == 'maverick' else 'Scout'} layer sizes, random bf16 weights)",
        "value": ns.batch / ms * 1e3, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0, 0.02), uniform random token ids, cache pre-filled with random keys and values",
        "config": {"model": f"llama4-{ns.preset}-sizes", "layers": ns.layers, "layers_full_model": SCOUT_FULL_LAYERS,
                   "hidden": cfg.hidden_size, "q_heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "experts": cfg.num_local_experts, "expert_inter": cfg.intermediate_size,
                   "shared_inter": cfg.intermediate_size, "vocab": cfg.vocab_size, "chunk": cfg.attention_chunk_size,
                   "global_batch": ns.batch, "seq_len": ns.context, "page_size": page, "parallelism": "single-gpu",
                   "l2": "inputs larger than L2 (weights and cache read per step exceed 126 MB many times over)"},
        "e2e": {"value": ns.batch / e2e_ms * 1e3, "unit": "tokens/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "bytes_per_step": need, "peak_kind": pk_kind,
                     "distinct_experts_per_layer": distinct},
        "points": points,
        "clocks": clock_summary,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
