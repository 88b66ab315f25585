"""``sharpi-cli``: the command line, with the reference's option names where it has them
(src/SharpInference.Cli/RunCommand.cs:25-297; app name and default command,
src/SharpInference.Cli/Program.cs:11-24).

Kept with the same spelling, meaning and default: ``-m|--model`` (here a model folder),
``-p|--prompt``, ``-f|--file``, ``-n|--n-predict`` (512), ``--temp`` (0.7; 0 = greedy), ``--top-k``
(40), ``--top-p`` (0.95), ``--min-p`` (0.05), ``-s|--seed`` (-1 = random), ``-c|--ctx-size``,
``--repeat-penalty`` (1.1), ``--repeat-last-n`` (256), ``--frequency-penalty``, ``--presence-penalty``,
``--verbose-prompt``, ``--no-display-prompt``, ``--device`` (an index or a name such as CUDA0; one GPU, and
no CPU), ``--min-batch-blas`` (the smallest step whose dense products go to the library's GEMM: below it the
engine's own weight-streaming kernel runs them, as the reference's matvec kernels do below its threshold,
src/SharpInference.Cli/RunCommand.cs:179-182; here 0 means the library at every size).  There is no tokenizer in this engine (random-weight
models have no vocabulary), so a prompt is a list of token ids: ``-p "5 17 3"`` or ``--tokens
5,17,3``; several prompts are separated by ``;`` and are served as one continuous batch.  Added:
``--dtype``, ``--random-weights SEED`` with ``--config`` (writes a model folder first),
``--max-batch``, ``--max-tokens-per-step``, ``--page-size``, ``--max-cache-tokens``.  The closing line
follows the reference's: ``Prefill: N tokens, X t/s | Decode: M tokens, Y t/s``
(src/SharpInference.Cli/RunCommand.cs:1907-1911).
"""
from __future__ import annotations

import argparse
import json
import re
import sys
import tempfile
import time
from typing import List


def parse_prompts(text: str) -> List[List[int]]:
    prompts = []
    for part in text.split(";"):
        ids = [int(t) for t in re.split(r"[\s,]+", part.strip()) if t]
        if ids:
            prompts.append(ids)
    return prompts


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="sharpi-cli", description="generate tokens with a model folder on one B200")
    ap.add_argument("command", nargs="?", default="run", choices=["run"], help="the default command")
    ap.add_argument("-m", "--model", help="model folder (config.json + model.safetensors)")
    ap.add_argument("-p", "--prompt", help="prompt as token ids, e.g. \"5 17 3\"; ';' separates prompts")
    ap.add_argument("-f", "--file", help="read the prompt (token ids) from a file; overrides -p")
    ap.add_argument("--tokens", help="prompt as comma-separated token ids (same as -p)")
    ap.add_argument("-n", "--n-predict", type=int, default=512, help="number of tokens to predict (default: 512)")
    ap.add_argument("--temp", type=float, default=0.7, help="temperature (0 = greedy, default: 0.7)")
    ap.add_argument("--top-k", type=int, default=40, help="top-k sampling (0 = disabled, default: 40)")
    ap.add_argument("--top-p", type=float, default=0.95, help="top-p nucleus sampling (default: 0.95)")
    ap.add_argument("--min-p", type=float, default=0.05, help="min-p sampling (default: 0.05)")
    ap.add_argument("-s", "--seed", type=int, default=-1, help="RNG seed (-1 = random, default: -1)")
    ap.add_argument("-c", "--ctx-size", type=int, default=0, help="context size (0 = model default)")
    ap.add_argument("--repeat-penalty", "--rep-penalty", type=float, default=1.1, dest="repeat_penalty")
    ap.add_argument("--repeat-last-n", type=int, default=256)
    ap.add_argument("--frequency-penalty", type=float, default=0.0)
    ap.add_argument("--presence-penalty", type=float, default=0.0)
    ap.add_argument("--verbose-prompt", action="store_true", help="print token ids before generating")
    ap.add_argument("--no-display-prompt", action="store_true", help="don't echo the prompt")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "bf16", "fp32"])
    ap.add_argument("--random-weights", type=int, default=None, metavar="SEED",
                    help="write a model folder with seeded random weights from --config first")
    ap.add_argument("--config", help="config.json for --random-weights")
    ap.add_argument("--max-batch", type=int, default=8)
    ap.add_argument("--max-tokens-per-step", type=int, default=2048)
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--max-cache-tokens", type=int, default=None)
    ap.add_argument("--device", default=None,
                    help="GPU to run on: an index (0, 1, ...) or a name (CUDA0, cuda:1); default: cuda:0.  One device "
                         "only; 'none' (CPU) is refused: the engine has no CPU path")
    ap.add_argument("--min-batch-blas", type=int, default=0,
                    help="smallest step (rows) whose dense products go to the library's GEMM; smaller steps run them on "
                         "the engine's own weight-streaming kernel (at most 17: that kernel takes up to 16 rows).  "
                         "0 (default): the library at every size, which is the faster step on B200")
    ap.add_argument("--json", action="store_true", help="print the result as one JSON object")
    ap.add_argument("--trace-layers", action="store_true",
                    help="after every step print, per layer, the L2 norm of the last row's residual and the expert "
                         "it was routed to (steps then run eagerly); for finding the first layer that differs")
    return ap


def parse_device(text):
    """``--device`` in the reference's spellings (src/SharpInference.Cli/RunCommand.cs:99-102: an index, or a name
    such as CUDA0) and torch's; None for anything else, 'none' (CPU) included."""
    if text is None or text == "" or text.lower() == "auto":
        return "cuda:0"
    t = text.strip().lower()
    for prefix in ("cuda:", "cuda", ""):
        if t.startswith(prefix) and t[len(prefix):].isdigit():
            return f"cuda:{int(t[len(prefix):])}"
    return None


def main(argv=None) -> int:
    ns = build_parser().parse_args(argv)
    text = ns.tokens or ns.prompt
    if ns.file:
        with open(ns.file, "r", encoding="utf-8") as fh:
            text = fh.read()
    if not text:
        print("sharpi-cli: give a prompt as token ids with -p, --tokens or -f", file=sys.stderr)
        return 2
    prompts = parse_prompts(text)

    from . import Engine, EngineOptions, SamplingParams, write_random_model

    model_dir = ns.model
    tmp = None
    if ns.random_weights is not None:
        if not ns.config:
            print("sharpi-cli: --random-weights needs --config FILE", file=sys.stderr)
            return 2
        with open(ns.config, "r", encoding="utf-8") as fh:
            cfg = json.load(fh)
        tmp = tempfile.TemporaryDirectory(prefix="sharpi_random_")
        model_dir = write_random_model(cfg, ns.model or tmp.name, ns.random_weights)
    if not model_dir:
        print("sharpi-cli: give a model folder with -m (or --random-weights SEED --config FILE)", file=sys.stderr)
        return 2

    cache_tokens = ns.max_cache_tokens
    if cache_tokens is None and ns.ctx_size > 0:
        cache_tokens = ns.ctx_size * ns.max_batch
    device = parse_device(ns.device)
    if device is None:
        print(f"sharpi-cli: --device {ns.device!r}: expected an index, CUDA<n> or cuda:<n> (the engine has no CPU path)",
              file=sys.stderr)
        return 2
    engine = Engine(model_dir, dtype=ns.dtype, device=device, options=EngineOptions(
        page_size=ns.page_size, max_cache_tokens=cache_tokens, max_batch=ns.max_batch,
        max_tokens_per_step=ns.max_tokens_per_step, own_dense_rows=max(0, min(ns.min_batch_blas, 17) - 1)))
    params = [SamplingParams(temperature=ns.temp, top_k=ns.top_k, top_p=ns.top_p, min_p=ns.min_p,
                             repetition_penalty=ns.repeat_penalty, penalty_last_n=ns.repeat_last_n,
                             frequency_penalty=ns.frequency_penalty, presence_penalty=ns.presence_penalty,
                             max_new_tokens=ns.n_predict, seed=(ns.seed + i) if ns.seed >= 0 else None)
              for i in range(len(prompts))]
    if ns.verbose_prompt:
        for i, p in enumerate(prompts):
            print(f"prompt {i}: {len(p)} tokens: {p}", file=sys.stderr)

    import torch
    ids = [engine.add_request(p, sp) for p, sp in zip(prompts, params)]
    prefill_tokens = sum(len(p) for p in prompts)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    t_first = None
    if ns.trace_layers:
        engine.runner.trace_layers = engine.runner.trace_router = True
    steps = 0
    while engine.has_unfinished:
        engine.step()
        if ns.trace_layers:
            picks = iter(engine.runner.last_router_choices)
            for layer, norms in enumerate(engine.runner.last_layer_norms):
                block = engine.model.blocks[engine.model.schedule[layer].layer]
                routed = getattr(getattr(block, "ffn", None), "num_experts", 0) > 0
                expert = int(next(picks)[-1]) if routed else None
                print(f"step {steps} layer {layer}: |x| = {float(norms[-1]):.6f}"
                      + (f", expert {expert}" if expert is not None else ""), file=sys.stderr)
        steps += 1
        if t_first is None and all(engine.output(i).tokens or engine.output(i).finished for i in ids):
            torch.cuda.synchronize()
            t_first = time.perf_counter()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    outs = [engine.output(i) for i in ids]
    decode_tokens = sum(max(len(o.tokens) - 1, 0) for o in outs)
    if ns.json:
        print(json.dumps({"outputs": [{"prompt": o.prompt, "tokens": o.tokens, "finish_reason": o.finish_reason}
                                      for o in outs]}))
    else:
        for o in outs:
            if not ns.no_display_prompt:
                print(" ".join(map(str, o.prompt)), end=" | ")
            print(" ".join(map(str, o.tokens)))
    t_first = t_first or t1
    pre_s, dec_s = max(t_first - t0, 1e-9), max(t1 - t_first, 1e-9)
    print(f"Prefill: {prefill_tokens} tokens, {prefill_tokens / pre_s:.1f} t/s | "
          f"Decode: {decode_tokens} tokens, {decode_tokens / dec_s:.1f} t/s", file=sys.stderr)
    if tmp is not None:
        tmp.cleanup()
    return 0


if __name__ == "__main__":
    sys.exit(main())
