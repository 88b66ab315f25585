"""Generality of the parts: a toy mixer with state of its own, a toy feed-forward that routes rows
between two sub-networks and a toy position encoding that is no rotation, all defined here, are
registered, built into toy architectures and stepped through the unchanged framework; and a schedule
that names a layer twice and lets a layer read another's cache (needs a GPU).  Nothing here is a
model of anyone's: the toy parts exist to exercise the interfaces."""
import json
import os
from dataclasses import asdict, dataclass

import pytest
import torch

import plain_llama4 as plain
import traces
from conftest import TINY_A, TINY_A_INIT

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


# ---------------------------------------------------------------------------------------
# a mixer with state: s <- decay * s + h_t ; out_t = W s
# ---------------------------------------------------------------------------------------
def define_toy():
    from sharpinference_b200.models.model import DecoderModel
    from sharpinference_b200.parts import (DenseSwiGLU, Linear, PagedAttention, PreNormBlock, RMSNorm,
                                           RotaryEncoding, rotary_inv_freq)
    from sharpinference_b200.parts.base import Mixer, StateSpec, make_part, register_part
    from sharpinference_b200.registry import register_architecture

    @register_part("mixer", "toy_decay")
    class DecayMixer(Mixer):
        def __init__(self, *, weight, decay, act_dtype):
            self.weight, self.decay, self.act_dtype = weight, float(decay), act_dtype
            self.state_spec = StateSpec((weight.shape[1],), torch.float32)
            self.cache_spec = None

        def forward(self, ctx, slot, h):
            out = torch.empty((ctx.num_tokens, self.weight.shape[0]), dtype=torch.float32, device=h.device)
            row = 0
            for b in range(ctx.num_requests):
                s = slot.state[ctx.host_state_slots[b]]
                for _ in range(ctx.host_lengths[b]):
                    s.mul_(self.decay).add_(h[row].float())
                    out[row] = self.weight.float() @ s
                    row += 1
            return out

    @dataclass(frozen=True)
    class ToyConfig:
        vocab_size: int = 50
        hidden_size: int = 40
        intermediate_size: int = 56
        num_heads: int = 5
        head_dim: int = 16
        window: int = 6
        decay: float = 0.75
        eps: float = 1e-5
        architecture = "ToyDecayForCausalLM"

        @classmethod
        def from_dict(cls, obj, where="config.json"):
            return cls(**{k: obj[k] for k in cls.__dataclass_fields__ if k in obj})

        def to_dict(self):
            return {"architectures": [self.architecture], **asdict(self)}

    def build(c, weights):
        act, H, I = weights.compute_dtype, c.hidden_size, c.intermediate_size

        def ffn(p):
            return DenseSwiGLU(gate_up=Linear(weights.matrix(p + "gate_up.weight", (2 * I, H))),
                               down=Linear(weights.matrix(p + "down.weight", (H, I))), act_dtype=act)

        def norm(name):
            return RMSNorm(weights.vector(name, (H,)), c.eps)

        inv = rotary_inv_freq(c.head_dim, 100.0, None)
        inv = inv if weights.device.type == "meta" else inv.to(weights.device)
        blocks = [
            PreNormBlock(mixer_norm=norm("l0.n1"), ffn_norm=norm("l0.n2"), ffn=ffn("l0."), act_dtype=act,
                         mixer=make_part("mixer", "toy_decay", weight=weights.matrix("l0.mix.weight", (H, H)),
                                         decay=c.decay, act_dtype=act)),
            PreNormBlock(mixer_norm=norm("l1.n1"), ffn_norm=norm("l1.n2"), ffn=ffn("l1."), act_dtype=act,
                         mixer=PagedAttention(qkv=Linear(weights.matrix("l1.qkv.weight", (3 * c.num_heads * c.head_dim, H))),
                                              out=Linear(weights.matrix("l1.o.weight", (H, c.num_heads * c.head_dim))),
                                              num_heads=c.num_heads, num_kv_heads=c.num_heads, head_dim=c.head_dim,
                                              mask="window", span=c.window, position=RotaryEncoding(inv, "halves"),
                                              act_dtype=act)),
        ]
        return DecoderModel(embedding=weights.matrix("embed.weight", (c.vocab_size, H)), blocks=blocks,
                            final_norm=norm("final.weight"), head=Linear(weights.matrix("head.weight", (c.vocab_size, H))),
                            act_dtype=act, config=c)

    register_architecture("ToyDecayForCausalLM", ToyConfig, build)
    return ToyConfig


def toy_plain(folder, toks):
    """Whole-sequence statement of the toy model in float64."""
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as fh:
        c = json.load(fh)
    w = {k: v.double() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    H, nh, d, S = c["hidden_size"], c["num_heads"], c["head_dim"], len(toks)
    x = w["embed.weight"][torch.tensor(toks)]
    h = plain.rms_norm(x, w["l0.n1"], c["eps"])
    s, mixed = torch.zeros(H, dtype=torch.float64), []
    for t in range(S):
        s = c["decay"] * s + h[t]
        mixed.append(w["l0.mix.weight"] @ s)
    x = x + torch.stack(mixed)
    def ffn(p, h):
        gu = h @ w[p + "gate_up.weight"].T
        return (plain.silu(gu[:, :c["intermediate_size"]]) * gu[:, c["intermediate_size"]:]) @ w[p + "down.weight"].T
    x = x + ffn("l0.", plain.rms_norm(x, w["l0.n2"], c["eps"]))
    h = plain.rms_norm(x, w["l1.n1"], c["eps"])
    qkv = (h @ w["l1.qkv.weight"].T)
    q, k, v = (qkv[:, i * nh * d:(i + 1) * nh * d].reshape(S, nh, d) for i in range(3))
    inv = 1.0 / torch.pow(torch.tensor(100.0), torch.arange(d // 2, dtype=torch.float32) * 2.0 / d)
    ang = (torch.arange(S).float()[:, None] * inv[None, :]).double()
    cs, sn = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    rot = lambda z: torch.cat([z[..., :d // 2] * cs - z[..., d // 2:] * sn, z[..., :d // 2] * sn + z[..., d // 2:] * cs], -1)
    x = x + plain.attention_scores(rot(q), rot(k), v, plain.visible("window", c["window"], S)) @ w["l1.o.weight"].T
    x = x + ffn("l1.", plain.rms_norm(x, w["l1.n2"], c["eps"]))
    return plain.rms_norm(x, w["final.weight"], c["eps"]) @ w["head.weight"].T


@pytest.fixture(scope="module")
def toy_folder(tmp_path_factory):
    from sharpinference_b200 import write_random_model
    ToyConfig = define_toy()
    out = str(tmp_path_factory.mktemp("toy"))
    write_random_model(ToyConfig(), out, seed=11, std=0.15, norm_std=0.1)
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_is_built_and_stepped(toy_folder, dtype):
    from sharpinference_b200 import Engine, EngineOptions
    reqs = {f"t{i}": traces.random_tokens(50, n, seed=n) for i, n in enumerate([30, 9, 41, 17, 25])}
    ref = {rid: toy_plain(toy_folder, toks) for rid, toks in reqs.items()}
    for cut in (traces.whole, traces.portions, lambda r: traces.mixed(r, max_live=2)):
        steps = cut(reqs)
        eng = Engine(toy_folder, dtype=dtype, device=DEV,
                     options=EngineOptions(page_size=4, max_cache_tokens=traces.max_tokens(steps), max_batch=2))
        assert [g.spec.kind for g in eng.cache.groups] == ["window"]
        state = eng.cache.layer_slots()[0].state
        assert state is not None and state.shape == (2, 40)
        got = traces.replay(eng, steps)
        err, where = traces.worst_error(got, ref)
        assert err < (2e-5 if dtype == "float32" else 3e-2), (err, where)
        # with two state slots and five requests, slots were reused: a stale state would have shown
        assert not eng.cache.requests and eng.cache.state_slots.free_count == 2


def test_toy_generation_through_the_scheduler(toy_folder):
    from sharpinference_b200 import Engine, EngineOptions, SamplingParams
    prompts = [traces.random_tokens(50, n, seed=n + 1) for n in (12, 3, 20)]
    eng = Engine(toy_folder, dtype="float32", device=DEV,
                 options=EngineOptions(page_size=4, max_cache_tokens=256, max_batch=3, max_tokens_per_step=7))
    got = eng.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=5))
    for p, g in zip(prompts, got):
        seq = list(p)
        for tok in g:
            assert plain.greedy(toy_plain(toy_folder, seq)[-1]) == tok
            seq.append(tok)


# ---------------------------------------------------------------------------------------
# a feed-forward that routes, and a position encoding that adds instead of rotating
# ---------------------------------------------------------------------------------------
def define_routed_toy():
    from sharpinference_b200.models.model import DecoderModel
    from sharpinference_b200.parts import DenseSwiGLU, Linear, PagedAttention, PreNormBlock, RMSNorm
    from sharpinference_b200.parts.base import FeedForward, PositionEncoding, make_part, register_part
    from sharpinference_b200.registry import register_architecture

    @register_part("position", "toy_additive")
    class AdditiveWaves(PositionEncoding):
        """q += amp * sin(pos * f), k += amp * cos(pos * f): positions enter by addition, not rotation."""
        def __init__(self, freqs, amp):
            self.freqs, self.amp = freqs, float(amp)

        def apply(self, ctx, q, k):
            angle = ctx.positions.to(torch.float32)[:, None] * self.freqs[None, :]          # [T, d]
            q.add_(self.amp * torch.sin(angle)[:, None, :])
            k.add_(self.amp * torch.cos(angle)[:, None, :])

    @register_part("feed_forward", "toy_sign_route")
    class SignRouted(FeedForward):
        """Rows whose projection on a direction is positive go through one network, the others through
        another; the output is scaled by tanh of the projection."""
        wants_fp32_input = True

        def __init__(self, *, direction, positive, negative):
            self.direction, self.positive, self.negative = direction, positive, negative

        def forward(self, ctx, h, h32=None):
            h32 = h.float() if h32 is None else h32
            score = h32 @ self.direction.float()
            out = torch.zeros((h.shape[0], self.positive.down.out_features), dtype=torch.float32, device=h.device)
            for net, rows in ((self.positive, (score > 0).nonzero().flatten()), (self.negative, (score <= 0).nonzero().flatten())):
                if rows.numel():
                    out[rows] = net.forward(ctx, h[rows].contiguous())
            return out * torch.tanh(score)[:, None]

    @dataclass(frozen=True)
    class RoutedToyConfig:
        vocab_size: int = 37
        hidden_size: int = 24
        intermediate_size: int = 40
        num_heads: int = 3
        num_kv_heads: int = 1
        head_dim: int = 16
        num_layers: int = 2
        amp: float = 0.4
        eps: float = 1e-4
        architecture = "ToyRoutedForCausalLM"

        @classmethod
        def from_dict(cls, obj, where="config.json"):
            return cls(**{k: obj[k] for k in cls.__dataclass_fields__ if k in obj})

        def to_dict(self):
            return {"architectures": [self.architecture], **asdict(self)}

    def build(c, weights):
        act, H, I, d = weights.compute_dtype, c.hidden_size, c.intermediate_size, c.head_dim
        freqs = 0.3 * torch.arange(1, d + 1, dtype=torch.float32)
        freqs = freqs if weights.device.type == "meta" else freqs.to(weights.device)

        def ffn(p):
            return DenseSwiGLU(gate_up=Linear(weights.matrix(p + "gate_up.weight", (2 * I, H))),
                               down=Linear(weights.matrix(p + "down.weight", (H, I))), act_dtype=act)

        def norm(name):
            return RMSNorm(weights.vector(name, (H,)), c.eps)

        blocks = []
        for i in range(c.num_layers):
            p = f"l{i}."
            mixer = PagedAttention(qkv=Linear(weights.matrix(p + "qkv.weight", ((c.num_heads + 2 * c.num_kv_heads) * d, H))),
                                   out=Linear(weights.matrix(p + "o.weight", (H, c.num_heads * d))),
                                   num_heads=c.num_heads, num_kv_heads=c.num_kv_heads, head_dim=d, mask="full",
                                   position=make_part("position", "toy_additive", freqs=freqs, amp=c.amp), act_dtype=act)
            routed = make_part("feed_forward", "toy_sign_route", direction=weights.vector(p + "route", (H,)),
                               positive=ffn(p + "pos."), negative=ffn(p + "neg."))
            blocks.append(PreNormBlock(mixer_norm=norm(p + "n1"), ffn_norm=norm(p + "n2"), ffn=routed, act_dtype=act, mixer=mixer))
        return DecoderModel(embedding=weights.matrix("embed.weight", (c.vocab_size, H)), blocks=blocks,
                            final_norm=norm("final.weight"), head=Linear(weights.matrix("head.weight", (c.vocab_size, H))),
                            act_dtype=act, config=c)

    register_architecture("ToyRoutedForCausalLM", RoutedToyConfig, build)
    return RoutedToyConfig


def routed_toy_plain(folder, toks, amp=None):
    """Whole-sequence statement of the routed toy model in float64; also the smallest |routing score|."""
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as fh:
        c = json.load(fh)
    if amp is not None:
        c["amp"] = amp
    w = {k: v.double() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    nq, nkv, d, S, I = c["num_heads"], c["num_kv_heads"], c["head_dim"], len(toks), c["intermediate_size"]
    x = w["embed.weight"][torch.tensor(toks)]
    angle = torch.arange(S, dtype=torch.float64)[:, None] * (0.3 * torch.arange(1, d + 1, dtype=torch.float32)).double()[None, :]
    margin = float("inf")
    for i in range(c["num_layers"]):
        p = f"l{i}."
        h = plain.rms_norm(x, w[p + "n1"], c["eps"])
        qkv = h @ w[p + "qkv.weight"].T
        q = qkv[:, : nq * d].reshape(S, nq, d) + c["amp"] * torch.sin(angle)[:, None, :]
        k = qkv[:, nq * d: (nq + nkv) * d].reshape(S, nkv, d) + c["amp"] * torch.cos(angle)[:, None, :]
        v = qkv[:, (nq + nkv) * d:].reshape(S, nkv, d)
        x = x + plain.attention_scores(q, k, v, plain.visible("full", 0, S)) @ w[p + "o.weight"].T
        h = plain.rms_norm(x, w[p + "n2"], c["eps"])
        score = h @ w[p + "route"]
        margin = min(margin, float(score.abs().min()))
        y = torch.zeros_like(x)
        for name, rows in (("pos.", score > 0), ("neg.", score <= 0)):
            gu = h[rows] @ w[p + name + "gate_up.weight"].T
            y[rows] = (plain.silu(gu[:, :I]) * gu[:, I:]) @ w[p + name + "down.weight"].T
        x = x + y * torch.tanh(score)[:, None]
    return plain.rms_norm(x, w["final.weight"], c["eps"]) @ w["head.weight"].T, margin


def test_toy_routing_feed_forward_and_additive_positions(tmp_path):
    """A feed-forward that routes rows and a position encoding that is no rotation, defined in this file,
    run through the unchanged engine: whole, in portions and mixed with page reuse, against the plain
    statement.  (float32: a routing score near zero may fall the other way in bfloat16.)"""
    from sharpinference_b200 import Engine, EngineOptions, write_random_model
    from sharpinference_b200.registry import unregister_architecture
    Cfg = define_routed_toy()
    try:
        folder = str(tmp_path / "routed")
        write_random_model(Cfg(), folder, seed=5, std=0.2, norm_std=0.1)
        reqs = {f"q{i}": traces.random_tokens(37, n, seed=3 * n) for i, n in enumerate([33, 6, 45, 12])}
        ref, margins = {}, []
        for rid, toks in reqs.items():
            ref[rid], m = routed_toy_plain(folder, toks)
            margins.append(m)
        assert min(margins) > 1e-4          # no row sits on the routing boundary
        for cut in (traces.whole, traces.portions, lambda r: traces.mixed(r, max_live=3)):
            steps = cut(reqs)
            eng = Engine(folder, dtype="float32", device=DEV,
                         options=EngineOptions(page_size=4, max_cache_tokens=traces.max_tokens(steps), max_batch=3))
            got = traces.replay(eng, steps)
            err, where = traces.worst_error(got, ref)
            assert err < 2e-5, (err, where)
        # the encoding is really applied: without it the plain statement gives other logits
        without, _ = routed_toy_plain(folder, reqs["q0"], amp=0.0)
        assert float((without - ref["q0"]).abs().max()) > 1e-3
    finally:
        unregister_architecture("ToyRoutedForCausalLM")


# ---------------------------------------------------------------------------------------
# the schedule as data
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_layer_named_twice_and_a_borrowed_cache(tmp_path, dtype):
    from sharpinference_b200 import Engine, EngineOptions, write_random_model
    from sharpinference_b200.config import Llama4TextConfig
    from sharpinference_b200.models.llama4 import build_llama4
    from sharpinference_b200.models.model import ScheduleEntry
    from sharpinference_b200.registry import register_architecture, unregister_architecture

    order = [(0, None), (1, None), (2, None), (1, None), (3, None), (2, 2), (3, 4)]

    def build(config, weights):
        return build_llama4(config, weights).set_schedule([ScheduleEntry(layer, borrow) for layer, borrow in order])

    class Cfg(Llama4TextConfig):
        architecture = "Llama4TwiceForCausalLM"

        def to_dict(self):
            return dict(super().to_dict(), architectures=[self.architecture])

    register_architecture("Llama4TwiceForCausalLM", Cfg, build)
    try:
        folder = str(tmp_path / "m")
        write_random_model(dict(TINY_A, architectures=["Llama4TwiceForCausalLM"]), folder, 3, std=0.05, norm_std=0.1)
        cfg, w = plain.load_folder(folder)
        reqs = {f"r{i}": traces.random_tokens(cfg["vocab_size"], n, seed=n) for i, n in enumerate([37, 50, 8])}
        steps = traces.mixed(reqs, max_live=2)
        eng = Engine(folder, dtype=dtype, device=DEV,
                     options=EngineOptions(page_size=8, max_cache_tokens=traces.max_tokens(steps), max_batch=2))
        # seven schedule entries; two of them borrow, so five caches in two groups
        assert sorted(len(g.entries) for g in eng.cache.groups) == [1, 4]
        routing = {} if dtype == "bfloat16" else None
        got = traces.replay(eng, steps, routing)
        ref = {rid: plain.forward(cfg, w, toks, schedule=order, forced=None if routing is None else routing[rid])
               for rid, toks in reqs.items()}
        err, where = traces.worst_error(got, ref)
        assert err < (2e-5 if dtype == "float32" else 3e-2), (err, where)
    finally:
        unregister_architecture("Llama4TwiceForCausalLM")


def test_schedule_is_validated():
    from sharpinference_b200.models.model import DecoderModel, ScheduleEntry
    from sharpinference_b200.weights import DeclaringWeights
    from sharpinference_b200.config import Llama4TextConfig
    from sharpinference_b200.models.llama4 import build_llama4
    model = build_llama4(Llama4TextConfig.from_dict(TINY_A), DeclaringWeights())
    with pytest.raises(ValueError, match="names block 9"):
        model.set_schedule([ScheduleEntry(9)])
    with pytest.raises(ValueError, match="must come earlier"):
        model.set_schedule([ScheduleEntry(0, cache_from=0)])
    with pytest.raises(ValueError, match="cache needs differ"):
        model.set_schedule([ScheduleEntry(0), ScheduleEntry(3, cache_from=0)])      # chunked against full
    with pytest.raises(ValueError, match="itself borrows"):
        model.set_schedule([ScheduleEntry(0), ScheduleEntry(1, cache_from=0), ScheduleEntry(2, cache_from=1)])


# ---------------------------------------------------------------------------------------
# a mixer that ships per-step metadata of its own and is replayed inside a captured decode graph
# ---------------------------------------------------------------------------------------
def define_prefix_toy():
    """out_t = W . mean(h_0 .. h_t): a running sum per request in a state slot.  Within a step the sums are a
    segmented prefix sum over the step's rows, for which the mixer needs to know, per row, where its request's
    rows begin, and per request, which row is its last: metadata that its own planner adds to the step.  It
    reads the step through device tensors only, so decode steps with it are captured and replayed."""
    import numpy as np
    from sharpinference_b200.models.model import DecoderModel
    from sharpinference_b200.parts import DenseSwiGLU, Linear, PreNormBlock, RMSNorm
    from sharpinference_b200.parts.base import Mixer, StateSpec, StepPlanData, StepPlanner, make_part, register_part
    from sharpinference_b200.registry import register_architecture

    class SegmentPlanner(StepPlanner):
        key = "toy_segments"

        def plan(self, starts, lengths, bucket=None):
            first = np.cumsum([0] + list(lengths[:-1]))
            return StepPlanData(arrays={"row_first": np.repeat(first, lengths), "last_row": first + np.asarray(lengths) - 1},
                                values={"requests": len(lengths)})

    @register_part("mixer", "toy_prefix_mean")
    class PrefixMean(Mixer):
        graph_safe = True

        def __init__(self, *, weight, act_dtype):
            self.weight, self.act_dtype = weight, act_dtype
            self.state_spec = StateSpec((weight.shape[1],), torch.float32)
            self.cache_spec = None

        def step_planner(self, page_size):
            return SegmentPlanner()

        def forward(self, ctx, slot, h):
            plan = ctx.plans["toy_segments"]
            h32 = h.float()
            run = torch.cumsum(h32, dim=0)
            first = plan.row_first.long()
            within = run - (run[first] - h32[first])                       # inclusive sums inside each request's rows
            slots = ctx.state_slots.long()
            total = slot.state[slots[ctx.row_request.long()]] + within
            slot.state.index_copy_(0, slots, total[plan.last_row.long()])  # the state after the request's last row
            mean = total / (ctx.positions.float() + 1.0)[:, None]
            return mean @ self.weight.float().t()

    @dataclass(frozen=True)
    class PrefixToyConfig:
        vocab_size: int = 41
        hidden_size: int = 32
        intermediate_size: int = 48
        num_layers: int = 2
        eps: float = 1e-5
        architecture = "ToyPrefixForCausalLM"

        @classmethod
        def from_dict(cls, obj, where="config.json"):
            return cls(**{k: obj[k] for k in cls.__dataclass_fields__ if k in obj})

        def to_dict(self):
            return {"architectures": [self.architecture], **asdict(self)}

    def build(c, weights):
        act, H, I = weights.compute_dtype, c.hidden_size, c.intermediate_size
        norm = lambda name: RMSNorm(weights.vector(name, (H,)), c.eps)
        blocks = [PreNormBlock(mixer_norm=norm(f"l{i}.n1"), ffn_norm=norm(f"l{i}.n2"), act_dtype=act,
                               mixer=make_part("mixer", "toy_prefix_mean", weight=weights.matrix(f"l{i}.mix.weight", (H, H)),
                                               act_dtype=act),
                               ffn=DenseSwiGLU(gate_up=Linear(weights.matrix(f"l{i}.gate_up.weight", (2 * I, H))),
                                               down=Linear(weights.matrix(f"l{i}.down.weight", (H, I))), act_dtype=act))
                  for i in range(c.num_layers)]
        return DecoderModel(embedding=weights.matrix("embed.weight", (c.vocab_size, H)), blocks=blocks,
                            final_norm=norm("final.weight"), head=Linear(weights.matrix("head.weight", (c.vocab_size, H))),
                            act_dtype=act, config=c)

    register_architecture("ToyPrefixForCausalLM", PrefixToyConfig, build)
    return PrefixToyConfig


def prefix_toy_plain(folder, toks):
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as fh:
        c = json.load(fh)
    w = {k: v.double() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    I, S = c["intermediate_size"], len(toks)
    x = w["embed.weight"][torch.tensor(toks)]
    for i in range(c["num_layers"]):
        h = plain.rms_norm(x, w[f"l{i}.n1"], c["eps"])
        mean = torch.cumsum(h, 0) / torch.arange(1, S + 1, dtype=torch.float64)[:, None]
        x = x + mean @ w[f"l{i}.mix.weight"].T
        h = plain.rms_norm(x, w[f"l{i}.n2"], c["eps"])
        gu = h @ w[f"l{i}.gate_up.weight"].T
        x = x + (plain.silu(gu[:, :I]) * gu[:, I:]) @ w[f"l{i}.down.weight"].T
    return plain.rms_norm(x, w["final.weight"], c["eps"]) @ w["head.weight"].T


def test_toy_mixer_with_its_own_step_metadata_inside_a_decode_graph(tmp_path):
    """The planner and the mixer are defined above, in this file: the step function ships the planner's arrays
    without knowing what they mean, in eager steps and in the static buffer of a replayed graph alike."""
    from sharpinference_b200 import Engine, EngineOptions, write_random_model
    from sharpinference_b200.registry import unregister_architecture
    Cfg = define_prefix_toy()
    try:
        folder = str(tmp_path / "prefix")
        write_random_model(Cfg(), folder, seed=8, std=0.2, norm_std=0.1)
        reqs = {f"p{i}": traces.random_tokens(41, n, seed=5 * n) for i, n in enumerate([50, 23, 61, 9])}
        ref = {rid: prefix_toy_plain(folder, toks) for rid, toks in reqs.items()}
        # every way of cutting, in 32-bit
        for cut in (traces.whole, traces.portions, lambda r: traces.mixed(r, max_live=3), lambda r: traces.tail_decode(r, 32)):
            eng = Engine(folder, dtype="float32", device=DEV, options=EngineOptions(page_size=16, max_cache_tokens=64, max_batch=3))
            assert list(eng.runner.planners) == ["toy_segments"] and eng.runner.use_graphs and not eng.cache.groups
            got = traces.replay(eng, cut(reqs))
            err, where = traces.worst_error(got, ref)
            assert err < 2e-5, (err, where)
        assert eng.runner.graph_replays >= 3 * 28          # tail_decode: 32 single-token steps per request, replayed
        # three requests decode together, then two, then one: graphs of three shapes, same numbers as eager steps
        heads = {"p0": 20, "p1": 10, "p2": 5}
        steps = [{"step": 0, "entries": [{"id": r, "tokens": reqs[r][:n], "want": []} for r, n in heads.items()], "end": []}]
        at, s = dict(heads), 0
        while at:
            s += 1
            entries = [{"id": r, "tokens": [reqs[r][p]], "want": [0]} for r, p in at.items()]
            at = {r: p + 1 for r, p in at.items()}
            ended = [r for r, p in at.items() if p == len(reqs[r])]
            steps.append({"step": s, "entries": entries, "end": ended})
            for r in ended:
                del at[r]
        outs = {}
        for graphs in (False, True):
            eng = Engine(folder, dtype="float32", device=DEV,
                         options=EngineOptions(page_size=16, max_cache_tokens=64, max_batch=3, cuda_graphs=graphs))
            outs[graphs] = traces.replay(eng, steps)
            assert (eng.runner.graph_replays > 40) == graphs
        for key, row in outs[False].items():
            assert torch.equal(row, outs[True][key]), key
        err, where = traces.worst_error(outs[True], ref)
        assert err < 2e-5, (err, where)
    finally:
        unregister_architecture("ToyPrefixForCausalLM")
