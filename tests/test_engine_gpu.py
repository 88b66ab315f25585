"""The engine against the plain implementation under every way of cutting the work, in 32-bit and
in bfloat16 (needs a GPU)."""
import os

import pytest
import torch

import plain_llama4 as plain
import traces
from conftest import LARGE_SHAPES, REAL_WIDTHS, TINY

pytestmark = pytest.mark.gpu

# Error budgets, relative to the largest |logit| of the request.  float32: every product and sum
# is 32-bit with at most a few hundred terms, six layers deep.  bfloat16: activations and
# weights enter each matrix product rounded to 8 bits of mantissa (2^-9 relative), products
# accumulate in 32-bit, the residual stream, norms, softmax and router stay 32-bit.
TOL = {"float32": 2e-5, "bfloat16": 2e-2}
# Top-1 routing is discontinuous: where two experts' gate values are closer than bfloat16
# rounding can resolve, the engine may send a token to the other one, and then its logits differ
# by far more than rounding although nothing is wrong.  The bfloat16 comparisons therefore run
# the plain implementation with the engine's expert choices and require that every differing
# choice was such a near-tie: its gate value lies within MARGIN of the largest one.
MARGIN = 4e-3
LENGTHS = {"A": [5, 17, 40, 70], "B": [1, 9, 33, 70, 100], "C": [3, 50, 61], "D": [130, 7, 75]}


def requests_for(name):
    vocab = TINY[name][0]["vocab_size"]
    return {f"r{i}": traces.random_tokens(vocab, n, seed=100 * i + n) for i, n in enumerate(LENGTHS[name])}


@pytest.fixture(scope="module")
def expected(model_dirs):
    out = {}
    for name in TINY:
        cfg, w = plain.load_folder(model_dirs[name])
        out[name] = {rid: plain.forward(cfg, w, toks) for rid, toks in requests_for(name).items()}
    return out


def plain_under_engine_routing(model_dir, reqs, routing, dtype=torch.float64, margin=MARGIN):
    """Plain logits per request with the engine's expert choices imposed; asserts near-ties."""
    cfg, w = plain.load_folder(model_dir, dtype)
    ref, flips = {}, 0
    for rid, toks in reqs.items():
        margins = []
        ref[rid] = plain.forward(cfg, w, toks, forced=routing.get(rid), margins=margins)
        for layer in margins:
            assert max(layer, default=0.0) < margin, f"request {rid}: an expert choice differs beyond a near-tie"
            flips += sum(m > 0 for m in layer)
    return ref, flips


def near_tie_margin(model_dir):
    """What counts as a near-tie of two gate values at a model's own scale.  A gate is the sigmoid of a router
    logit, whose slope is at most 1/4; the router's input has unit mean square, so its logits are of the size of
    a router row's norm; and the engine's bfloat16 logits are held to TOL of their scale everywhere else.  So two
    gates closer than TOL / 4 of a router row's norm are closer than the engine can tell apart.  For the tiny
    models that is less than MARGIN, which stays their bound; at the large models' width (rows of 5120 weights of
    0.02: norm 1.43) it is 7e-3, and choices that differ by up to 6e-3 do occur there."""
    cfg, w = plain.load_folder(model_dir, torch.float32)
    rows = [float(t.norm(dim=1).mean()) for name, t in w.items() if name.endswith("feed_forward.router.weight")]
    return max(MARGIN, 0.25 * TOL["bfloat16"] * max(rows, default=0.0))


def make_engine(model_dir, dtype, max_tokens, page_size=16):
    from sharpinference_b200 import Engine, EngineOptions
    return Engine(model_dir, dtype=dtype, device="cuda:0",
                  options=EngineOptions(page_size=page_size, max_cache_tokens=max_tokens, max_batch=8))


CUTS = {
    "whole": traces.whole,
    "tail_decode": traces.tail_decode,
    "portions": traces.portions,
    "mixed": traces.mixed,
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cut", list(CUTS))
@pytest.mark.parametrize("name", list(TINY))
def test_logits_equal_the_plain_implementation(model_dirs, expected, name, cut, dtype):
    reqs = requests_for(name)
    steps = CUTS[cut](reqs)
    engine = make_engine(model_dirs[name], dtype, traces.max_tokens(steps, page=16))      # not a page to spare
    routing = {} if dtype == "bfloat16" else None
    got = traces.replay(engine, steps, routing)
    assert len(got) == sum(len(t) for t in reqs.values())
    ref, flips = (expected[name], 0) if routing is None else plain_under_engine_routing(model_dirs[name], reqs, routing)
    err, where = traces.worst_error(got, ref)
    print(f"{name} {cut} {dtype}: worst relative error {err:.3e} at {where}; near-tie expert choices: {flips}")
    assert err < TOL[dtype], f"worst error {err:.3e} at {where}"
    engine.cache.check_invariants()
    assert not engine.cache.requests
    assert all(g.pages.held_count == 0 for g in engine.cache.groups)


@pytest.fixture(scope="module")
def large_shapes(tmp_path_factory):
    from sharpinference_b200.weights import write_random_model
    folder = str(tmp_path_factory.mktemp("large_shapes"))
    write_random_model(dict(LARGE_SHAPES), folder, 4, std=0.03, norm_std=0.1)
    reqs = {f"L{i}": traces.random_tokens(1000, n, seed=31 * i + n) for i, n in enumerate([1400, 300, 77, 650])}
    return folder, reqs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cut", ["whole", "tail_decode", "mixed"])
def test_large_model_shapes_in_small(large_shapes, cut, dtype):
    from sharpinference_b200 import Engine, EngineOptions
    folder, reqs = large_shapes
    steps = CUTS[cut](reqs)
    engine = Engine(folder, dtype=dtype, device="cuda:0",
                    options=EngineOptions(page_size=64, max_cache_tokens=traces.max_tokens(steps), max_batch=8))
    if dtype == "bfloat16":
        assert ("paged_attention", 128) in engine.runner.planners          # the tcgen05 attention kernel serves the prompts
    routing = {} if dtype == "bfloat16" else None
    got = traces.replay(engine, steps, routing)
    if routing is None:
        cfg, w = plain.load_folder(folder)
        ref, flips = {rid: plain.forward(cfg, w, toks) for rid, toks in reqs.items()}, 0
    else:
        ref, flips = plain_under_engine_routing(folder, reqs, routing)
    err, where = traces.worst_error(got, ref)
    print(f"large shapes {cut} {dtype}: worst relative error {err:.3e} at {where}; near-tie expert choices: {flips}")
    assert err < TOL[dtype], f"worst error {err:.3e} at {where}"
    engine.cache.check_invariants()
    assert all(g.pages.held_count == 0 for g in engine.cache.groups)


@pytest.fixture(scope="module")
def real_widths(tmp_path_factory):
    from sharpinference_b200.weights import write_random_model
    folder = str(tmp_path_factory.mktemp("real_widths"))
    write_random_model(dict(REAL_WIDTHS), folder, 5, std=0.02, norm_std=0.1)
    reqs = {f"W{i}": traces.random_tokens(2048, n, seed=17 * i + n) for i, n in enumerate([1100, 40, 300])}
    return folder, reqs


@pytest.mark.parametrize("cut", ["tail_decode", "mixed"])
def test_layer_widths_of_the_large_models(real_widths, cut):
    """Hidden 5120, 40/8 heads of 128, experts of 8192, a dense layer of 16384: the kernels at the sizes the
    benchmarks run them at (the persistent expert product for the 1100-token prompt, K cut over CTAs for the
    decoded tokens), against the plain implementation in 32-bit on the same bfloat16 weights."""
    from sharpinference_b200 import Engine, EngineOptions
    folder, reqs = real_widths
    steps = CUTS[cut](reqs)
    engine = Engine(folder, dtype="bfloat16", device="cuda:0",
                    options=EngineOptions(page_size=64, max_cache_tokens=traces.max_tokens(steps), max_batch=8))
    routing = {}
    got = traces.replay(engine, steps, routing)
    ref, flips = plain_under_engine_routing(folder, reqs, routing, dtype=torch.float32, margin=near_tie_margin(folder))
    err, where = traces.worst_error(got, ref)
    print(f"real widths {cut}: worst relative error {err:.3e} at {where}; near-tie expert choices: {flips}")
    assert err < TOL["bfloat16"], f"worst error {err:.3e} at {where}"
    engine.cache.check_invariants()
    assert all(g.pages.held_count == 0 for g in engine.cache.groups)


@pytest.mark.parametrize("rows", [8, 16])
def test_dense_products_on_the_engines_own_kernel(large_shapes, rows):
    """own_dense_rows: decode-size steps run their dense products (qkv, o, shared expert, dense layers) on the
    weight-streaming kernel up to that many rows (16: its wide form too) instead of the library; the LM head
    stays on the library; the logits stay within rounding."""
    from sharpinference_b200 import Engine, EngineOptions
    folder, reqs = large_shapes
    reqs = {k: v[:200] for k, v in list(reqs.items())[:3]}
    steps = traces.tail_decode(reqs)
    engine = Engine(folder, dtype="bfloat16", device="cuda:0",
                    options=EngineOptions(page_size=64, max_cache_tokens=traces.max_tokens(steps), max_batch=8,
                                          own_dense_rows=rows))
    assert all(b.mixer.qkv.stream_rows == rows and b.ffn.shared.gate_up.stream_rows == rows for b in engine.model.blocks)
    assert engine.model.head.stream_rows == 0
    routing = {}
    got = traces.replay(engine, steps, routing)
    ref, _ = plain_under_engine_routing(folder, reqs, routing)
    err, where = traces.worst_error(got, ref)
    assert err < TOL["bfloat16"], (err, where)


@pytest.mark.parametrize("name", list(TINY))
def test_float32_cuts_agree_with_each_other_tightly(model_dirs, name):
    """In 32-bit every kernel sums in an order that depends on the row alone, so a row's logits
    are the same numbers however the work is cut (up to the last bits of exp and division)."""
    reqs = requests_for(name)
    runs = {}
    for cut in ("whole", "portions", "mixed"):
        steps = CUTS[cut](reqs)
        runs[cut] = traces.replay(make_engine(model_dirs[name], "float32", traces.max_tokens(steps)), steps)
    for key, row in runs["whole"].items():
        for cut in ("portions", "mixed"):
            assert torch.allclose(row, runs[cut][key], rtol=0, atol=1e-6 * float(row.abs().max())), (cut, key)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pages_are_really_used_again(model_dirs, dtype):
    """Mixed trace over eight requests with a pool sized for three: every page goes out more than once."""
    name = "B"
    cfg, w = plain.load_folder(model_dirs[name])
    reqs = {f"q{i}": traces.random_tokens(cfg["vocab_size"], n, seed=7 * i + n)
            for i, n in enumerate([40, 55, 70, 33, 64, 48, 90, 20])}
    ref = {rid: plain.forward(cfg, w, toks) for rid, toks in reqs.items()}
    steps = traces.mixed(reqs, max_live=3)
    engine = make_engine(model_dirs[name], dtype, traces.max_tokens(steps, page=16), page_size=16)
    taken = {g.index: 0 for g in engine.cache.groups}
    for g in engine.cache.groups:
        def counting(g=g, inner=g.pages.take):
            taken[g.index] += 1
            return inner()
        g.pages.take = counting
    routing = {} if dtype == "bfloat16" else None
    got = traces.replay(engine, steps, routing)
    if routing is not None:
        ref, _ = plain_under_engine_routing(model_dirs[name], reqs, routing)
    err, where = traces.worst_error(got, ref)
    print(f"page reuse {dtype}: worst relative error {err:.3e} at {where}")
    assert err < TOL[dtype], (err, where)
    assert len(engine.cache.groups) == 2
    for g in engine.cache.groups:                     # the chunked group and the one that keeps everything
        assert taken[g.index] > g.pages.capacity, f"group {g.index} ({g.spec.kind}): no page went out twice"
    assert all(g.pages.held_count == 0 for g in engine.cache.groups)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decode_and_first_tokens(model_dirs, dtype):
    """A request decoded token by token from its very first token, across several chunks."""
    name = "A"
    cfg, w = plain.load_folder(model_dirs[name])
    toks = traces.random_tokens(cfg["vocab_size"], 150, seed=9)
    ref = {"x": plain.forward(cfg, w, toks)}
    steps = [{"step": i, "entries": [{"id": "x", "tokens": [t], "want": [0]}], "end": ["x"] if i == len(toks) - 1 else []}
             for i, t in enumerate(toks)]
    engine = make_engine(model_dirs[name], dtype, 192, page_size=16)
    routing = {} if dtype == "bfloat16" else None
    got = traces.replay(engine, steps, routing)
    if routing is not None:
        ref, _ = plain_under_engine_routing(model_dirs[name], {"x": toks}, routing)
    err, where = traces.worst_error(got, ref)
    print(f"long decode {dtype}: worst relative error {err:.3e} at {where}")
    assert err < TOL[dtype], (err, where)
    # the chunked group never held more than a chunk (16 positions = 1 page) plus the page being written
    first = {k: v for k, v in got.items() if k[1] < 3}
    e3, _ = traces.worst_error(first, ref)
    assert e3 < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(model_dirs, name, dtype):
    from sharpinference_b200 import Engine, EngineOptions, SamplingParams
    cfg, w = plain.load_folder(model_dirs[name])
    prompts = [traces.random_tokens(cfg["vocab_size"], n, seed=n) for n in (5, 17, 40)]
    want = [plain.generate_greedy(cfg, w, p, 8) for p in prompts]
    engine = Engine(model_dirs[name], dtype=dtype, device="cuda:0",
                    options=EngineOptions(page_size=16, max_cache_tokens=256, max_batch=4, max_tokens_per_step=24))
    got = engine.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=8))
    if dtype == "float32":
        assert got == want
    else:
        # a near-tie may fall the other way in bfloat16; after that the sequences differ
        # legitimately, so compare up to the first difference and require it to be a near-tie
        for p, g, x in zip(prompts, got, want):
            for i, (a, b) in enumerate(zip(g, x)):
                if a != b:
                    row = plain.forward(cfg, w, p + x[:i])[-1]
                    assert float(row[b] - row[a]) < 3e-2 * float(row.abs().max()), (i, a, b)
                    break
    assert not engine.cache.requests


def test_generation_with_preemption_gives_the_same_tokens(model_dirs):
    """So few pages that a running request is preempted and recomputed: same tokens."""
    from sharpinference_b200 import Engine, EngineOptions, SamplingParams
    cfg, w = plain.load_folder(model_dirs["A"])
    prompts = [traces.random_tokens(cfg["vocab_size"], n, seed=n) for n in (20, 22, 18)]
    want = [plain.generate_greedy(cfg, w, p, 12) for p in prompts]
    engine = Engine(model_dirs["A"], dtype="float32", device="cuda:0",
                    options=EngineOptions(page_size=8, max_cache_tokens=72, max_batch=3, max_tokens_per_step=32))
    got = engine.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=12))
    assert got == want
    assert engine.scheduler.num_preemptions >= 1
    assert not engine.cache.requests
    m = engine.metrics()
    assert m["queued"] == 0 and m["running"] == 0 and m["preemptions"] == engine.scheduler.num_preemptions
    assert all(g["free"] == g["pages"] == 9 and g["held"] == 0 for g in m["cache_groups"].values())
    # every prompt token and all but each request's last new token went through a step, some of them twice
    assert m["decode_tokens"] + m["prefill_tokens"] >= 60 + 3 * 11 and m["prefill_tokens"] >= 60 and m["steps"] > 12


def test_temperature_sampling_is_reproducible_and_follows_the_distribution(model_dirs):
    from sharpinference_b200 import Engine, EngineOptions, SamplingParams
    from sharpinference_b200.sampling import uniform01
    cfg, w = plain.load_folder(model_dirs["B"])
    prompts = [traces.random_tokens(cfg["vocab_size"], n, seed=n) for n in (1, 9, 33)]
    sp = SamplingParams(temperature=0.8, max_new_tokens=6, seed=1234)

    def run(max_tokens_per_step):
        engine = Engine(model_dirs["B"], dtype="float32", device="cuda:0",
                        options=EngineOptions(page_size=16, max_cache_tokens=512, max_batch=4,
                                              max_tokens_per_step=max_tokens_per_step))
        return engine.generate(prompts, sp)

    a, b = run(64), run(7)
    assert a == b                              # the same seed draws the same tokens in any batching
    # and they are the tokens the plain sampler draws from the plain logits with the same numbers
    for p, out in zip(prompts, a):
        seq = list(p)
        for n, tok in enumerate(out):
            dist = plain.sample_distribution(plain.forward(cfg, w, seq)[-1], 0.8)
            assert plain.draw(dist, uniform01(1234, n)) == tok
            seq.append(tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_steps_replayed_as_cuda_graphs_give_the_same_logits(model_dirs, dtype):
    """Decode-only steps are captured per shape and replayed; the numbers must be those of eager steps,
    also when the batch changes shape and when a request's block table grows past the captured width."""
    from sharpinference_b200 import Engine, EngineOptions
    name = "B"
    cfg, w = plain.load_folder(model_dirs[name])
    reqs = {f"g{i}": traces.random_tokens(cfg["vocab_size"], n, seed=50 + i) for i, n in enumerate([300, 280, 40])}
    # whole prompts first, then token by token: three live, then two, then one
    steps, s = [], 0
    heads = {"g0": 20, "g1": 10, "g2": 5}
    steps.append({"step": s, "entries": [{"id": r, "tokens": t[:heads[r]], "want": []} for r, t in reqs.items()], "end": []})
    at = dict(heads)
    while at:
        s += 1
        entries = [{"id": r, "tokens": [reqs[r][p]], "want": [0]} for r, p in at.items()]
        at = {r: p + 1 for r, p in at.items()}
        ended = [r for r, p in at.items() if p == len(reqs[r])]
        steps.append({"step": s, "entries": entries, "end": ended})
        for r in ended:
            del at[r]
    outs, routing = {}, {} if dtype == "bfloat16" else None
    for graphs in (False, True):
        eng = Engine(model_dirs[name], dtype=dtype, device="cuda:0",
                     options=EngineOptions(page_size=16, max_cache_tokens=traces.max_tokens(steps), max_batch=4,
                                           cuda_graphs=graphs))
        outs[graphs] = traces.replay(eng, steps, None if graphs else routing)     # the eager run records the experts
        assert (eng.runner.graph_replays > 200) == graphs
        assert not graphs or len(eng.runner._graphs) >= 4       # three batch shapes, and a wider table for the long ones
    for key, row in outs[False].items():
        assert torch.equal(row, outs[True][key]), key
    ref = ({rid: plain.forward(cfg, w, toks) for rid, toks in reqs.items()} if routing is None
           else plain_under_engine_routing(model_dirs[name], reqs, routing)[0])
    err, where = traces.worst_error(outs[True], ref)
    assert err < TOL[dtype], (err, where)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replayed_decode_steps_with_one_long_request_among_short_ones(model_dirs, dtype):
    """Four requests decode together, one with 880 keys and three with a few: the decode attention launch then
    counts all rows' splits together (in bfloat16), inside a replayed graph too; same numbers as eager steps."""
    from sharpinference_b200 import Engine, EngineOptions
    name = "D"                                   # head size 64: the split-KV kernels serve it in bfloat16
    cfg, w = plain.load_folder(model_dirs[name])
    reqs = {f"m{i}": traces.random_tokens(cfg["vocab_size"], n, seed=70 + i) for i, n in enumerate([900, 40, 30, 25])}
    heads = {"m0": 880, "m1": 20, "m2": 10, "m3": 5}
    steps = [{"step": 0, "entries": [{"id": r, "tokens": t[:heads[r]], "want": []} for r, t in reqs.items()], "end": []}]
    for s in range(1, 21):
        steps.append({"step": s, "entries": [{"id": r, "tokens": [reqs[r][heads[r] + s - 1]], "want": [0]} for r in reqs],
                      "end": list(reqs) if s == 20 else []})
    outs, routing = {}, {} if dtype == "bfloat16" else None
    for graphs in (False, True):
        eng = Engine(model_dirs[name], dtype=dtype, device="cuda:0",
                     options=EngineOptions(page_size=16, max_cache_tokens=traces.max_tokens(steps), max_batch=4,
                                           cuda_graphs=graphs))
        outs[graphs] = traces.replay(eng, steps, None if graphs else routing)
        assert (eng.runner.graph_replays >= 15) == graphs
    for key, row in outs[False].items():
        assert torch.equal(row, outs[True][key]), key
    cut = {rid: toks[:heads[rid] + 20] for rid, toks in reqs.items()}
    ref = ({rid: plain.forward(cfg, w, toks) for rid, toks in cut.items()} if routing is None
           else plain_under_engine_routing(model_dirs[name], cut, routing)[0])
    err, where = traces.worst_error(outs[True], ref)
    assert err < TOL[dtype], (err, where)


def test_sampling_options_through_the_entry_point(model_dirs):
    """top-k / top-p / min-p / penalties / logit bias / stop tokens as request parameters."""
    from sharpinference_b200 import Engine, EngineOptions, SamplingParams
    cfg, w = plain.load_folder(model_dirs["A"])
    eng = Engine(model_dirs["A"], dtype="float32", device="cuda:0",
                 options=EngineOptions(page_size=16, max_cache_tokens=512, max_batch=4, max_tokens_per_step=32))
    prompt = traces.random_tokens(cfg["vocab_size"], 12, seed=77)
    greedy = eng.generate([prompt], SamplingParams(temperature=0.0, max_new_tokens=6))[0]
    # top_k = 1 is greedy whatever the temperature and the seed
    assert eng.generate([prompt], SamplingParams(temperature=1.5, top_k=1, max_new_tokens=6, seed=5))[0] == greedy
    # a logit bias large enough forces its token (top_k = 1 makes the draw certain); greedy rows take the
    # arg-max of the raw logits before any bias or penalty, as the reference does
    forced = eng.generate([prompt], SamplingParams(temperature=1.0, top_k=1, max_new_tokens=3, logit_bias={7: 1e4}, seed=3))[0]
    assert forced == [7, 7, 7]
    assert eng.generate([prompt], SamplingParams(temperature=0.0, max_new_tokens=6, logit_bias={7: 1e4},
                                                 presence_penalty=1e4))[0] == greedy
    stopped = eng.generate([prompt], SamplingParams(temperature=0.0, max_new_tokens=6, stop_token_ids=[greedy[2]]))[0]
    assert stopped == greedy[:2]
    # a presence penalty that large forbids every token seen so far (prompt tail included)
    out = eng.generate([prompt], SamplingParams(temperature=1.0, top_k=1, max_new_tokens=10, presence_penalty=1e4, seed=4))[0]
    assert len(set(out)) == len(out) and not (set(out) & set(prompt))
    # nucleus sampling only ever returns tokens of the nucleus
    sp = SamplingParams(temperature=1.0, top_p=0.3, max_new_tokens=1, seed=11)
    dist = plain.sample_distribution(plain.forward(cfg, w, prompt)[-1], 1.0, top_p=0.3)
    for seed in range(20):
        tok = eng.generate([prompt], SamplingParams(temperature=1.0, top_p=0.3, max_new_tokens=1, seed=seed))[0][0]
        assert dist[tok] > 0
    assert not eng.cache.requests


def test_command_line_generates(model_dirs, tmp_path):
    import json
    import subprocess
    from conftest import ROOT, TINY_B
    cfg, w = plain.load_folder(model_dirs["B"])
    cli = os.path.join(ROOT, "bin", "sharpi-cli")
    proc = subprocess.run([cli, "-m", model_dirs["B"], "-p", "5 17 3; 9 9 200 1", "-n", "5", "--temp", "0", "--dtype",
                           "float32", "--page-size", "16", "--max-cache-tokens", "256", "--repeat-penalty", "1.0",
                           "--json"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr
    outs = json.loads(proc.stdout.strip().splitlines()[-1])["outputs"]
    assert [o["tokens"] for o in outs] == [plain.generate_greedy(cfg, w, p, 5) for p in ([5, 17, 3], [9, 9, 200, 1])]
    assert "Prefill: 7 tokens" in proc.stderr and "Decode: 8 tokens" in proc.stderr
    # random-weights mode: a config file and a seed are enough
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(TINY_B))
    proc = subprocess.run([cli, "--random-weights", "3", "--config", str(cfg_path), "--tokens", "1,2,3", "-n", "4",
                           "--temp", "0.8", "-s", "9", "--max-cache-tokens", "128", "--device", "CUDA0",
                           "--min-batch-blas", "9"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr
    assert len(proc.stdout.strip().splitlines()[-1].split("|")[-1].split()) == 4
    # --trace-layers: a line per step and layer, with the expert where the layer is a mixture (layers 1, 3, 5 of B)
    proc = subprocess.run([cli, "-m", model_dirs["B"], "-p", "5 17 3", "-n", "2", "--temp", "0", "--page-size", "16",
                           "--max-cache-tokens", "128", "--trace-layers"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr
    lines = [ln for ln in proc.stderr.splitlines() if ln.startswith("step ")]
    assert len(lines) == 2 * TINY_B["num_hidden_layers"]
    assert "step 0 layer 1: |x| = " in proc.stderr and ", expert " in lines[1] and ", expert " not in lines[0]


def random_configuration(seed: int) -> dict:
    """A configuration drawn from everything the architecture's config.json may say: head sizes in steps of
    16 (and one that is merely even), any heads and groups, widths and vocabularies that are no power of two,
    layers of both kinds of attention and both kinds of feed-forward in any arrangement."""
    import random
    r = random.Random(seed)
    nkv = r.choice([1, 2, 3])
    nq = nkv * r.choice([1, 2, 3, 5])
    d = r.choice([16, 32, 48, 64, 80, 96, 112, 128, 24])
    layers = r.randint(2, 5)
    hidden = r.choice([8 * r.randint(5, 20), 2 * r.randint(21, 60) + 2])          # the second: no multiple of 8
    chunk = 16 * r.randint(1, 4)
    scaling = None
    if r.random() < 0.5:
        scaling = {"rope_type": "llama3", "factor": r.choice([2.0, 8.0, 16.0]), "low_freq_factor": 1.0,
                   "high_freq_factor": r.choice([1.0, 4.0]), "original_max_position_embeddings": r.choice([16, 24, 64])}
    cfg = {
        "architectures": ["Llama4ForCausalLM"], "model_type": "llama4_text",
        "vocab_size": r.randint(100, 500) | 1, "hidden_size": hidden, "num_hidden_layers": layers,
        "num_attention_heads": nq, "num_key_value_heads": nkv, "head_dim": d,
        "intermediate_size": r.choice([8 * r.randint(3, 17), 2 * r.randint(13, 40) + 2]),
        "intermediate_size_mlp": 8 * r.randint(4, 30),
        "num_local_experts": r.randint(1, 9), "num_experts_per_tok": 1, "interleave_moe_layer_step": r.choice([1, 2]),
        "rope_theta": r.choice([1000.0, 10000.0, 500000.0]), "rope_scaling": scaling,
        "no_rope_layers": sorted(r.sample(range(layers), r.randint(0, layers))),
        "attention_chunk_size": chunk, "use_qk_norm": r.random() < 0.5, "qk_norm_eps": r.choice([1e-6, 1e-5]),
        "attn_temperature_tuning": r.random() < 0.5, "floor_scale": r.randint(3, 40), "attn_scale": r.choice([0.1, 0.3]),
        "rms_norm_eps": r.choice([1e-6, 1e-5, 1e-4]), "tie_word_embeddings": r.random() < 0.3,
    }
    if r.random() < 0.3:
        cfg["moe_layers"] = sorted(r.sample(range(layers), r.randint(0, layers)))
    return cfg


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(24))
def test_random_configurations(tmp_path, seed, dtype):
    """Drawn configurations, mixed batches on a cache so small that pages are used again."""
    from sharpinference_b200.weights import write_random_model
    cfg = random_configuration(seed)
    folder = str(tmp_path / "model")
    write_random_model(dict(cfg), folder, 50 + seed, std=0.06, norm_std=0.1)
    reqs = {f"q{i}": traces.random_tokens(cfg["vocab_size"], n, seed=7 * seed + n) for i, n in enumerate([3, 37, 90, 20, 55])}
    steps = traces.mixed(reqs)
    engine = make_engine(folder, dtype, traces.max_tokens(steps, page=16))
    routing = {} if dtype == "bfloat16" else None
    got = traces.replay(engine, steps, routing)
    if routing is None:
        pc, w = plain.load_folder(folder)
        ref, flips = {rid: plain.forward(pc, w, toks) for rid, toks in reqs.items()}, 0
    else:
        ref, flips = plain_under_engine_routing(folder, reqs, routing)
    err, where = traces.worst_error(got, ref)
    print(f"random configuration {seed} {dtype}: {cfg}\n  worst relative error {err:.3e} at {where}; near ties: {flips}")
    assert err < TOL[dtype], f"worst error {err:.3e} at {where} with {cfg}"
    engine.cache.check_invariants()
    assert all(g.pages.held_count == 0 for g in engine.cache.groups)


@pytest.mark.parametrize("seed", range(100, 108))
def test_random_configurations_on_the_tensor_memory_attention(tmp_path, seed):
    """Drawn configurations with head sizes 64 and 128 and pages of 64 positions, which is what the tcgen05
    attention kernel for prompts takes; prompts long enough for several of its tiles, chunks of one to four pages."""
    import random
    from sharpinference_b200 import Engine, EngineOptions
    from sharpinference_b200.weights import write_random_model
    r = random.Random(seed)
    cfg = random_configuration(seed)
    cfg["head_dim"] = r.choice([64, 128])
    cfg["attention_chunk_size"] = 64 * r.randint(1, 4)
    cfg["hidden_size"] = 8 * r.randint(5, 20)
    cfg["intermediate_size"] = 8 * r.randint(3, 17)
    folder = str(tmp_path / "model")
    write_random_model(dict(cfg), folder, seed, std=0.06, norm_std=0.1)
    reqs = {f"q{i}": traces.random_tokens(cfg["vocab_size"], n, seed=seed + n) for i, n in enumerate([300, 130, 70])}
    for cut in ("whole", "tail_decode"):
        steps = CUTS[cut](reqs)
        engine = Engine(folder, dtype="bfloat16", device="cuda:0",
                        options=EngineOptions(page_size=64, max_cache_tokens=traces.max_tokens(steps), max_batch=8))
        assert ("paged_attention", 128) in engine.runner.planners
        routing = {}
        got = traces.replay(engine, steps, routing)
        ref, flips = plain_under_engine_routing(folder, reqs, routing)
        err, where = traces.worst_error(got, ref)
        print(f"random configuration {seed} {cut}: {cfg}\n  worst relative error {err:.3e} at {where}; near ties: {flips}")
        assert err < TOL["bfloat16"], f"worst error {err:.3e} at {where} with {cfg}"
        engine.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(16))
def test_drawn_schedules(model_dirs, expected, seed, dtype):
    """Schedules drawn at random (who is live, who sits out, portion sizes, wanted places) on a cache that
    holds no more than the schedule needs at its fullest."""
    name = "ABCD"[seed % 4]
    reqs = requests_for(name)
    steps = traces.drawn(reqs, seed)
    engine = make_engine(model_dirs[name], dtype, traces.max_tokens(steps, page=16))
    routing = {} if dtype == "bfloat16" else None
    got = traces.replay(engine, steps, routing)
    ref, flips = (expected[name], 0) if routing is None else plain_under_engine_routing(model_dirs[name], reqs, routing)
    err, where = traces.worst_error(got, ref)
    print(f"{name} drawn schedule {seed} {dtype}: {len(steps)} steps, worst relative error {err:.3e} at {where}")
    assert err < TOL[dtype], f"worst error {err:.3e} at {where}"
    engine.cache.check_invariants()
    assert not engine.cache.requests
    assert all(g.pages.held_count == 0 for g in engine.cache.groups)


@pytest.mark.parametrize("name", ["A", "B"])
def test_layer_trace_follows_the_plain_implementation(model_dirs, name):
    """trace_layers: the residual's L2 norm per row after every layer, for finding the first layer that
    differs; in 32-bit it equals the plain implementation's layer by layer."""
    from sharpinference_b200 import StepEntry
    toks = requests_for(name)["r2"]
    engine = make_engine(model_dirs[name], "float32", 128)
    engine.runner.trace_layers = True
    engine.open_request("t")
    engine.forward_step([StepEntry("t", toks[:-3], [])])
    first = [n.cpu() for n in engine.runner.last_layer_norms]
    engine.forward_step([StepEntry("t", toks[-3:], [2])])
    second = [n.cpu() for n in engine.runner.last_layer_norms]
    engine.close_request("t")
    cfg, w = plain.load_folder(model_dirs[name])
    want = []
    plain.forward(cfg, w, toks, layer_norms=want)
    assert len(first) == len(second) == len(want) == cfg["num_hidden_layers"]
    for layer, ref in enumerate(want):
        got = torch.cat([first[layer], second[layer]]).double()
        assert torch.allclose(got, ref.double(), rtol=1e-5, atol=1e-6), f"layer {layer}"


# ---------------------------------------------------------------------------------------
# schedules: preemption with sampling and in bfloat16, abort in the middle of a prompt, graphs across a
# preemption, more decodes than the token budget
# ---------------------------------------------------------------------------------------
def same_or_near_tie(cfg, w, prompt, got, want, sp, seed=None):
    """The two token lists agree up to where bfloat16 rounding may decide otherwise: at the first difference
    both tokens must be all but equally likely for the plain implementation (a near-tie of the two logits for a
    greedy request; a draw that lies next to the border between the two tokens for a sampled one)."""
    from sharpinference_b200.sampling import uniform01
    for i, (a, b) in enumerate(zip(got, want)):
        if a == b:
            continue
        row = plain.forward(cfg, w, list(prompt) + list(want[:i]))[-1]
        if sp.temperature <= 0:
            assert abs(float(row[a] - row[b])) < 3e-2 * float(row.abs().max()), (i, a, b)
        else:
            dist = plain.sample_distribution(row, sp.temperature)
            u = uniform01(seed, i)
            near = {plain.draw(dist, min(max(u + e, 1e-7), 1 - 1e-7)) for e in (-0.03, -0.01, 0.0, 0.01, 0.03)}
            assert {a, b} <= near, (i, a, b, near)
        return
    assert len(got) == len(want)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sampling", ["greedy", "temperature"])
def test_preempted_requests_continue_where_they_were(model_dirs, dtype, sampling):
    """A cache so small that running requests are sent back and recomputed, against the same engine with room
    for all: the same tokens, also when they are drawn at a temperature (a request's random stream and output
    continue where they were)."""
    from sharpinference_b200 import Engine, EngineOptions, SamplingParams
    name = "B"
    cfg, w = plain.load_folder(model_dirs[name])
    prompts = [traces.random_tokens(cfg["vocab_size"], n, seed=40 + n) for n in (20, 22, 18, 9)]
    sp = SamplingParams(temperature=0.0 if sampling == "greedy" else 0.8, max_new_tokens=14, seed=77)

    def run(cache_tokens):
        eng = Engine(model_dirs[name], dtype=dtype, device="cuda:0",
                     options=EngineOptions(page_size=8, max_cache_tokens=cache_tokens, max_batch=4, max_tokens_per_step=32))
        out = eng.generate(prompts, sp)
        eng.cache.check_invariants()
        assert not eng.cache.requests and all(g.pages.held_count == 0 for g in eng.cache.groups)
        return out, eng.scheduler.num_preemptions

    want, none = run(512)
    got, some = run(80)
    assert none == 0 and some >= 1
    if dtype == "float32":
        assert got == want
    else:
        for p, g, x in zip(prompts, got, want):
            same_or_near_tie(cfg, w, p, g, x, sp, seed=77)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_abort_in_the_middle_of_a_prompt_and_the_pages_go_to_the_next_request(model_dirs, dtype):
    from sharpinference_b200 import Engine, EngineOptions, SamplingParams
    name = "A"
    cfg, w = plain.load_folder(model_dirs[name])
    eng = Engine(model_dirs[name], dtype=dtype, device="cuda:0",
                 options=EngineOptions(page_size=8, max_cache_tokens=64, max_batch=2, max_tokens_per_step=24))
    handed_out = {g.index: [] for g in eng.cache.groups}       # every page a group hands out, in order
    for g in eng.cache.groups:
        def noting(g=g, inner=g.pages.take):
            handed_out[g.index].append(inner())
            return handed_out[g.index][-1]
        g.pages.take = noting
    long_prompt = traces.random_tokens(cfg["vocab_size"], 60, seed=5)
    a = eng.add_request(long_prompt, SamplingParams(temperature=0.0, max_new_tokens=4))
    eng.step()                                            # 24 of the 60 tokens
    assert eng.request(a).computed == 24 and not eng.request(a).generated
    held = {gi: set(pages) for gi, pages in handed_out.items()}     # written by the request that is aborted now
    assert all(len(pages) == 3 for pages in held.values())
    for pages in handed_out.values():
        pages.clear()
    out = eng.abort(a)
    assert out.finish_reason == "abort" and not eng.cache.requests
    assert all(g.pages.held_count == 0 for g in eng.cache.groups)
    prompt = traces.random_tokens(cfg["vocab_size"], 50, seed=6)
    sp = SamplingParams(temperature=0.0, max_new_tokens=8)
    b = eng.add_request(prompt, sp)
    eng.step()
    reused = {gi: set(pages) & held[gi] for gi, pages in handed_out.items()}
    assert all(reused.values()), "the new request did not receive pages the aborted one had written"
    while eng.has_unfinished:
        eng.step()
    got, want = eng.output(b).tokens, plain.generate_greedy(cfg, w, prompt, 8)
    if dtype == "float32":
        assert got == want
    else:
        same_or_near_tie(cfg, w, prompt, got, want, sp)
    eng.cache.check_invariants()


def test_replayed_graphs_across_a_preemption(model_dirs):
    """Graphs on, and so few pages that a decoding request is sent back and admitted again between replays:
    the same ids return with new block tables.  Same tokens as eager steps on a cache with room for all."""
    from sharpinference_b200 import Engine, EngineOptions, SamplingParams
    name = "B"
    cfg, w = plain.load_folder(model_dirs[name])
    prompts = [traces.random_tokens(cfg["vocab_size"], n, seed=60 + n) for n in (12, 10, 14)]
    sp = SamplingParams(temperature=0.0, max_new_tokens=40)

    def run(cache_tokens, graphs):
        eng = Engine(model_dirs[name], dtype="float32", device="cuda:0",
                     options=EngineOptions(page_size=8, max_cache_tokens=cache_tokens, max_batch=3, max_tokens_per_step=32,
                                           cuda_graphs=graphs))
        out = eng.generate(prompts, sp)
        eng.cache.check_invariants()
        return out, eng.scheduler.num_preemptions, eng.runner.graph_replays

    want, _, zero = run(512, False)
    got, preemptions, replays = run(112, True)
    assert zero == 0 and preemptions >= 1 and replays >= 20
    assert got == want == [plain.generate_greedy(cfg, w, p, 40) for p in prompts]


def test_more_running_decodes_than_the_token_budget(model_dirs):
    from sharpinference_b200 import Engine, EngineOptions, SamplingParams
    name = "A"
    cfg, w = plain.load_folder(model_dirs[name])
    prompts = [traces.random_tokens(cfg["vocab_size"], n, seed=80 + i) for i, n in enumerate((3, 2, 3, 1, 2))]
    eng = Engine(model_dirs[name], dtype="float32", device="cuda:0",
                 options=EngineOptions(page_size=8, max_cache_tokens=256, max_batch=5, max_tokens_per_step=3))
    got = eng.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=9))
    assert got == [plain.generate_greedy(cfg, w, p, 9) for p in prompts]
    assert eng.runner.rows_run == sum(len(p) for p in prompts) + 5 * 8 and not eng.cache.requests


# ---------------------------------------------------------------------------------------
# the large models' mixtures and attention constants
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["16 experts", "128 experts"])
def test_sixteen_and_128_experts_through_the_engine(tmp_path_factory, which, dtype):
    from conftest import EXPERTS_16, EXPERTS_128
    from sharpinference_b200 import Engine, EngineOptions
    from sharpinference_b200.weights import write_random_model
    cfg = EXPERTS_16 if which == "16 experts" else EXPERTS_128
    folder = str(tmp_path_factory.mktemp("experts"))
    write_random_model(dict(cfg), folder, 21, std=0.03, norm_std=0.1)
    reqs = {f"E{i}": traces.random_tokens(1000, n, seed=13 * i + n) for i, n in enumerate([1300, 210, 66])}
    pc, w = plain.load_folder(folder)
    exact = {rid: plain.forward(pc, w, toks) for rid, toks in reqs.items()} if dtype == "float32" else None
    for cut in ("whole", "mixed"):
        steps = CUTS[cut](reqs)
        engine = Engine(folder, dtype=dtype, device="cuda:0",
                        options=EngineOptions(page_size=64, max_cache_tokens=traces.max_tokens(steps), max_batch=4))
        routing = {}
        got = traces.replay(engine, steps, routing)
        used = {e for layers in routing.values() for layer in layers for e in layer}
        assert len(used) > cfg["num_local_experts"] // 2          # the rows really spread over the experts
        ref = exact if exact is not None else plain_under_engine_routing(folder, reqs, routing)[0]
        err, where = traces.worst_error(got, ref)
        print(f"{which} {cut} {dtype}: worst relative error {err:.3e} at {where}; experts used: {len(used)}")
        assert err < TOL[dtype], f"worst error {err:.3e} at {where}"
        engine.cache.check_invariants()


@pytest.mark.parametrize("cut", ["whole", "portions"])
def test_layer_widths_of_the_large_models_whole_and_in_portions(real_widths, cut):
    from sharpinference_b200 import Engine, EngineOptions
    folder, reqs = real_widths
    reqs = {k: v[:700] for k, v in reqs.items()}
    steps = traces.whole(reqs) if cut == "whole" else traces.portions(reqs, sizes=(300, 2, 129, 64, 5, 200))
    engine = Engine(folder, dtype="bfloat16", device="cuda:0",
                    options=EngineOptions(page_size=64, max_cache_tokens=traces.max_tokens(steps), max_batch=8))
    routing = {}
    got = traces.replay(engine, steps, routing)
    ref, flips = plain_under_engine_routing(folder, reqs, routing, dtype=torch.float32, margin=near_tie_margin(folder))
    err, where = traces.worst_error(got, ref)
    print(f"real widths {cut}: worst relative error {err:.3e} at {where}; near-tie expert choices: {flips}")
    assert err < TOL["bfloat16"], f"worst error {err:.3e} at {where}"


def test_layer_widths_of_the_large_models_in_32_bit(real_widths):
    """The true 32-bit path at hidden 5120, 40/8 heads of 128, a dense layer of 16384 and experts of 8192 (the
    weights are the bfloat16 folder's, widened): a prompt, then its tail token by token, against the plain
    implementation in 64-bit."""
    from sharpinference_b200 import Engine, EngineOptions
    folder, reqs = real_widths
    reqs = {"W2": reqs["W2"][:150], "W1": reqs["W1"]}
    steps = traces.tail_decode(reqs, tail=8)
    engine = Engine(folder, dtype="float32", device="cuda:0",
                    options=EngineOptions(page_size=64, max_cache_tokens=traces.max_tokens(steps), max_batch=2))
    got = traces.replay(engine, steps)
    cfg, w = plain.load_folder(folder)
    ref = {rid: plain.forward(cfg, w, toks) for rid, toks in reqs.items()}
    err, where = traces.worst_error(got, ref)
    print(f"real widths float32: worst relative error {err:.3e} at {where}")
    assert err < TOL["float32"], f"worst error {err:.3e} at {where}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_request_crosses_the_edge_of_a_chunk_of_8192(tmp_path_factory, dtype):
    """attention_chunk_size = floor_scale = 8192 with pages of 64, as in the benchmark: a prompt of 8150 tokens
    in portions of 2048, then token by token to position 8300.  At 8192 the rotary layer's keys start over and
    the pages of its first chunk go back to the pool; from 8191 on the global layer's queries are scaled by
    1 + 0.1 ln 2.  A short request decodes beside it."""
    from conftest import CHUNK_EDGE
    from sharpinference_b200 import Engine, EngineOptions, StepEntry
    from sharpinference_b200.weights import write_random_model
    folder = str(tmp_path_factory.mktemp("chunk_edge"))
    write_random_model(dict(CHUNK_EDGE), folder, 31, std=0.08, norm_std=0.1)
    long_toks = traces.random_tokens(500, 8300, seed=1)
    short = traces.random_tokens(500, 170, seed=2)
    head = 8150
    engine = Engine(folder, dtype=dtype, device="cuda:0",
                    options=EngineOptions(page_size=64, max_cache_tokens=8320 + 192, max_batch=2))
    chunk = [g for g in engine.cache.groups if g.spec.kind == "chunk"][0]
    full = [g for g in engine.cache.groups if g.spec.kind == "full"][0]
    engine.runner.trace_router = dtype == "bfloat16"
    engine.open_request("long")
    engine.open_request("short")
    routing = {"long": [[]], "short": [[]]}
    got = {}

    def step(entries):
        logits = engine.forward_step([StepEntry(*e) for e in entries])
        if engine.runner.trace_router:
            picks, row = engine.runner.last_router_choices[0].cpu().tolist(), 0
            for rid, toks, _ in entries:
                routing[rid][0].extend(picks[row:row + len(toks)])
                row += len(toks)
        return None if logits is None else logits.float().cpu()

    at = 0
    while at < head:
        n = min(2048, head - at)
        step([("long", long_toks[at:at + n], [])])
        at += n
    step([("short", short[:20], [])])
    held_before = engine.cache.held_pages("long")
    assert held_before[chunk.index] == held_before[full.index] == (head + 63) // 64
    for i in range(head, 8300):
        j = 20 + (i - head)
        rows = step([("long", [long_toks[i]], [0]), ("short", [short[j]], [0])])
        got[("long", i)], got[("short", j)] = rows[0], rows[1]
        if i == 8192:
            held = engine.cache.held_pages("long")
            assert held[chunk.index] == 1 and held[full.index] == 8193 // 64 + 1      # the first chunk's pages are back
    engine.close_request("long")
    engine.close_request("short")
    engine.cache.check_invariants()
    pc, w = plain.load_folder(folder)
    reqs = {"long": long_toks, "short": short}
    forced = routing if dtype == "bfloat16" else {}
    ref = {rid: plain.forward(pc, w, toks, forced=forced.get(rid)) for rid, toks in reqs.items()}
    err, where = traces.worst_error(got, ref)
    print(f"chunk edge {dtype}: worst relative error {err:.3e} at {where}")
    assert err < TOL[dtype], f"worst error {err:.3e} at {where}"
    if dtype == "float32":
        # the test can see what it is there for: without the temperature factor, and with a chunk that does not
        # end at 8192, the plain implementation gives logits much further away than either tolerance
        after = [p for (rid, p) in got if rid == "long" and p >= 8192]
        w32 = {k: v.float() for k, v in w.items()}
        for change in ({"attn_temperature_tuning": False}, {"attention_chunk_size": 16384}):
            other = plain.forward(dict(pc, **change), w32, long_toks).double()
            scale = float(ref["long"].abs().max())
            gap = max(float((other[p] - ref["long"][p]).abs().max()) for p in after) / scale
            assert gap > 5 * TOL["bfloat16"], (change, gap)


def test_a_part_that_raises_in_mid_step_leaves_a_usable_engine(model_dirs):
    """A fault made on the host, inside the model: one layer's feed-forward raises once, in the middle of a step
    whose pages are reserved and whose first layers have run.  Every request of that moment ends with the error,
    their pages and slots come back, the captured graphs are dropped, and the same engine then generates what the
    plain implementation generates."""
    from sharpinference_b200 import Engine, EngineOptions, SamplingParams
    name = "A"
    cfg, w = plain.load_folder(model_dirs[name])
    eng = Engine(model_dirs[name], dtype="float32", device="cuda:0",
                 options=EngineOptions(page_size=8, max_cache_tokens=256, max_batch=3, max_tokens_per_step=32))
    prompts = [traces.random_tokens(cfg["vocab_size"], n, seed=90 + n) for n in (9, 14, 30, 5)]
    sp = SamplingParams(temperature=0.0, max_new_tokens=10)
    want = [plain.generate_greedy(cfg, w, p, 10) for p in prompts]
    assert eng.generate(prompts, sp) == want and eng.runner.graph_replays > 0 and eng.runner._graphs
    ffn = eng.model.blocks[2].ffn
    inner, calls = ffn.forward, {"n": 0}

    def flaky(ctx, h, h32=None):
        calls["n"] += 1
        if calls["n"] == 7:                              # some decode step
            raise RuntimeError("injected: this layer's feed-forward failed")
        return inner(ctx, h, h32)

    ffn.forward = flaky
    eng.runner.use_graphs = False                        # every step passes through the part above
    with pytest.raises(RuntimeError, match="injected"):
        eng.generate(prompts, sp)
    assert not eng.runner._graphs                        # the graphs captured before the failure are gone
    assert isinstance(eng.last_error, RuntimeError) and eng.stats["failed_steps"] == 1
    assert not eng.has_unfinished and not eng.cache.requests and not eng._requests
    assert all(g.pages.held_count == 0 for g in eng.cache.groups) and eng.cache.state_slots.free_count == 3
    eng.cache.check_invariants()
    errors = [eng.output(i) for i in list(eng._finished)]
    assert any(o.finish_reason == "error" and "injected" in o.error for o in errors)
    ffn.forward = inner
    eng.runner.use_graphs = True
    before = eng.runner.graph_replays
    assert eng.generate(prompts, sp) == want             # captured anew, in a new pool
    assert eng.runner.graph_replays > before and eng.runner._graphs


def test_cache_sized_from_free_memory_by_each_groups_needs(model_dirs):
    """Without max_cache_tokens the pool is sized from the device's free memory: the chunked group for max_batch
    requests of a chunk plus a step, the global group with the rest."""
    from sharpinference_b200 import Engine, EngineOptions, SamplingParams
    name = "B"
    cfg, w = plain.load_folder(model_dirs[name])
    eng = Engine(model_dirs[name], dtype="bfloat16", device="cuda:0",
                 options=EngineOptions(page_size=16, max_batch=4, max_tokens_per_step=64, memory_fraction=0.001))
    groups = {g.spec.kind: g for g in eng.cache.groups}
    assert groups["chunk"].pages.capacity == 4 * (32 + 64 + 16) // 16
    assert groups["full"].pages.capacity > 50 * groups["chunk"].pages.capacity
    prompt = traces.random_tokens(cfg["vocab_size"], 90, seed=12)
    sp = SamplingParams(temperature=0.0, max_new_tokens=5)
    same_or_near_tie(cfg, w, prompt, eng.generate([prompt], sp)[0], plain.generate_greedy(cfg, w, prompt, 5), sp)


def test_captured_graphs_are_evicted_and_captured_again(model_dirs):
    """Room for two graphs only, while the batch shrinks and grows: graphs are dropped oldest first and captured
    again when their shape returns; the logits stay those of eager steps."""
    from sharpinference_b200 import Engine, EngineOptions
    name = "A"
    cfg, w = plain.load_folder(model_dirs[name])
    reqs = {f"e{i}": traces.random_tokens(cfg["vocab_size"], 60, seed=200 + i) for i in range(3)}
    steps = [{"step": 0, "entries": [{"id": r, "tokens": t[:6], "want": []} for r, t in reqs.items()], "end": []}]
    at, s = {r: 6 for r in reqs}, 0
    while any(p < 60 for p in at.values()):
        s += 1
        live = [r for r in reqs if at[r] < 60 and (s // 4 + int(r[1])) % 3 != 0]      # who decodes changes every 4 steps
        if not live:
            continue
        steps.append({"step": s, "entries": [{"id": r, "tokens": [reqs[r][at[r]]], "want": [0]} for r in live], "end": []})
        for r in live:
            at[r] += 1
    steps[-1]["end"] = list(reqs)
    outs = {}
    for graphs in (False, True):
        eng = Engine(model_dirs[name], dtype="float32", device="cuda:0",
                     options=EngineOptions(page_size=16, max_cache_tokens=traces.max_tokens(steps), max_batch=4, cuda_graphs=graphs))
        eng.runner.max_graphs = 2
        outs[graphs] = traces.replay(eng, steps)
        if graphs:
            assert eng.runner.graph_replays > 30 and len(eng.runner._graphs) <= 2
    for key, row in outs[False].items():
        assert torch.equal(row, outs[True][key]), key
    ref = {rid: plain.forward(cfg, w, toks) for rid, toks in reqs.items()}
    err, where = traces.worst_error(outs[True], ref)
    assert err < TOL["float32"], (err, where)


@pytest.mark.parametrize("seed", range(3))
def test_random_arrivals_aborts_and_few_pages_through_the_entry_point(model_dirs, seed):
    """Requests arrive between steps, some are aborted at random moments, greedy and sampled ones side by side, on
    a cache and a token budget drawn small: after every step no page is lost or held twice, in the end everything
    is free, every request was reported once, and every greedy request that ran to its length has the plain
    implementation's tokens (32-bit)."""
    import random
    from sharpinference_b200 import Engine, EngineOptions, SamplingParams
    name = "ABD"[seed]
    cfg, w = plain.load_folder(model_dirs[name])
    rng = random.Random(seed)
    eng = Engine(model_dirs[name], dtype="float32", device="cuda:0",
                 options=EngineOptions(page_size=8, max_cache_tokens=rng.choice([96, 160]), max_batch=rng.choice([2, 4]),
                                       max_tokens_per_step=rng.choice([5, 16, 40])))
    pending = []
    for i in range(16):
        sp = SamplingParams(temperature=rng.choice([0.0, 0.0, 0.8]), max_new_tokens=rng.choice([1, 4, 9]),
                            seed=rng.randrange(1000), top_k=rng.choice([0, 0, 5]))
        pending.append((traces.random_tokens(cfg["vocab_size"], rng.choice([1, 2, 7, 19, 33, 60]), seed=100 * seed + i), sp))
    live, done, steps = {}, {}, 0
    while pending or eng.has_unfinished:
        if pending and rng.random() < 0.4:
            p, sp = pending.pop(0)
            live[eng.add_request(p, sp)] = (p, sp)
        if live and rng.random() < 0.05:
            rid = rng.choice(list(live))
            out = eng.abort(rid) if rid not in done else None
            if out is not None:
                done[rid] = out
        for out in eng.step():
            assert out.request_id not in done
            done[out.request_id] = out
        eng.cache.check_invariants()
        steps += 1
        assert steps < 3000
    assert not eng.cache.requests and all(g.pages.held_count == 0 for g in eng.cache.groups)
    assert eng.cache.state_slots.free_count == eng.cache.max_requests and set(done) == set(live) and not eng._requests
    checked = 0
    for rid, out in done.items():
        p, sp = live[rid]
        assert out.finished and out.finish_reason in ("length", "abort", "cache_full")
        if out.finish_reason == "length" and sp.temperature == 0.0:
            assert out.tokens == plain.generate_greedy(cfg, w, p, sp.max_new_tokens), (rid, out.preemptions)
            checked += 1
    assert checked >= 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(2))
def test_drawn_schedules_with_long_portions_at_the_large_models_shapes(large_shapes, seed, dtype):
    """Drawn schedules whose portions run from one token to 700 (around the 128-row attention tiles: 127, 128, 129)
    beside decoded tokens of other requests, at head size 128 and pages of 64: the tcgen05 attention with partial
    tiles, the split-KV kernel and every form of the grouped product in the same steps."""
    from sharpinference_b200 import Engine, EngineOptions
    folder, reqs = large_shapes
    steps = traces.drawn(reqs, seed, sizes=(1, 2, 3, 5, 17, 64, 127, 128, 129, 300, 700), want_share=0.2)
    engine = Engine(folder, dtype=dtype, device="cuda:0",
                    options=EngineOptions(page_size=64, max_cache_tokens=traces.max_tokens(steps), max_batch=4))
    routing = {} if dtype == "bfloat16" else None
    got = traces.replay(engine, steps, routing)
    if routing is None:
        cfg, w = plain.load_folder(folder)
        ref = {rid: plain.forward(cfg, w, toks) for rid, toks in reqs.items()}
    else:
        ref, _ = plain_under_engine_routing(folder, reqs, routing)
    err, where = traces.worst_error(got, ref)
    print(f"large shapes, drawn schedule {seed} {dtype}: {len(steps)} steps, worst relative error {err:.3e} at {where}")
    assert err < TOL[dtype], f"worst error {err:.3e} at {where}"
    engine.cache.check_invariants()
    assert all(g.pages.held_count == 0 for g in engine.cache.groups)
