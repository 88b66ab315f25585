"""The plain implementation itself (no GPU): small pins taken from the reference's own tests, and
properties that any correct implementation has."""
import math

import pytest
import torch

import plain_llama4 as plain
from conftest import TINY_A, TINY_B, TINY_C
from sharpinference_b200.config import Llama4TextConfig
from sharpinference_b200.parts.position import rotary_inv_freq


def test_rmsnorm_pin():
    # tests/SharpInference.Tests.ForwardPass/PipelineStepTests.cs:215-229: [1,2,3,4], w = 1, eps = 1e-5 -> x / sqrt(7.5)
    x = torch.tensor([1.0, 2.0, 3.0, 4.0], dtype=torch.float64)
    out = plain.rms_norm(x, torch.ones(4, dtype=torch.float64), 1e-5)
    assert torch.allclose(out, x / math.sqrt(7.5 + 1e-5), atol=1e-12)


def test_l2_norm_has_length_sqrt_dim():
    # PipelineStepTests.cs:282-302: the weightless norm's output has L2 norm sqrt(dim)
    x = torch.randn(5, 48, dtype=torch.float64)
    out = plain.l2_norm(x, 1e-12)
    assert torch.allclose(out.norm(dim=-1), torch.full((5,), math.sqrt(48.0), dtype=torch.float64), atol=1e-6)


def test_router_pin_sigmoid_then_first_max():
    # PipelineStepTests.cs:55-75, :136-149: 16 logits whose largest is index 11, sigmoid about 0.3
    logits = torch.full((16,), -2.0, dtype=torch.float64)
    logits[11] = -0.84
    logits[4] = -0.84          # an equal value later loses; earlier wins
    p = torch.sigmoid(logits)
    best, idx = p[0], 0
    for j in range(1, 16):
        if p[j] > best:
            best, idx = p[j], j
    assert idx == 4 and 0.299 < float(best) < 0.302


def test_greedy_lowest_index_wins_ties():
    # tests/SharpInference.Tests.ForwardPass/CudaGpuArgmaxParityTests.cs:84-100
    assert plain.greedy(torch.tensor([1.0, 5.0, 5.0, 2.0])) == 1
    assert plain.greedy(torch.tensor([3.0, 3.0, 3.0])) == 0


def test_weight_before_the_nonlinearity_is_not_weight_after():
    # PipelineStepTests.cs:184-208
    g, u, w = torch.tensor([0.7, -1.2]), torch.tensor([1.5, 0.3]), 0.3
    before = plain.silu(w * g) * (w * u)
    after = w * (plain.silu(g) * u)
    assert not torch.allclose(before, after)


@pytest.mark.parametrize("cfg", [TINY_A, TINY_B, TINY_C])
def test_rope_frequencies_agree_with_the_package(cfg):
    typed = Llama4TextConfig.from_dict(cfg)
    ours = rotary_inv_freq(typed.head_dim, typed.rope_theta, typed.rope_scaling)
    theirs = plain.rope_frequencies(cfg)
    assert torch.allclose(ours, theirs, rtol=3e-7, atol=0)


def test_llama3_scaling_cases():
    cfg = dict(TINY_B)
    f = plain.rope_frequencies(cfg)
    base = plain.rope_frequencies(dict(cfg, rope_scaling=None))
    L, low, high, factor = 16.0, 1.0, 4.0, 8.0
    for fj, bj in zip(f.tolist(), base.tolist()):
        ratio = L * bj / (2 * math.pi)
        if ratio > high:
            assert fj == pytest.approx(bj)
        elif ratio < low:
            assert fj == pytest.approx(bj / factor)
        else:
            assert bj / factor < fj < bj
    # low == high: a pure step (the Scout setting)
    step = plain.rope_frequencies(TINY_C)
    base_c = plain.rope_frequencies(dict(TINY_C, rope_scaling=None))
    for fj, bj in zip(step.tolist(), base_c.tolist()):
        assert fj == pytest.approx(bj) or fj == pytest.approx(bj / 4.0)


def test_rope_rotates_pairs_and_keeps_lengths():
    x = torch.randn(3, 2, 8, dtype=torch.float64)
    f = torch.tensor([1.0, 0.5, 0.25, 0.125])
    out = plain.apply_rope(x, torch.tensor([0, 1, 7]), f)
    assert torch.allclose(out[0], x[0])                                   # position 0: identity
    assert torch.allclose(out.norm(dim=-1), x.norm(dim=-1))
    a = 7 * 0.5
    x0, x1 = x[2, 1, 2], x[2, 1, 3]
    assert out[2, 1, 2] == pytest.approx(float(x0 * math.cos(a) - x1 * math.sin(a)))
    assert out[2, 1, 3] == pytest.approx(float(x0 * math.sin(a) + x1 * math.cos(a)))


def test_masks():
    ok = plain.visible("chunk", 4, 10)
    assert ok[5].tolist() == [False] * 4 + [True, True] + [False] * 4
    assert ok[4].tolist() == [False] * 4 + [True] + [False] * 5
    assert plain.visible("full", 0, 4)[2].tolist() == [True, True, True, False]
    assert plain.visible("window", 3, 6)[5].tolist() == [False, False, False, True, True, True]


def test_temperature_factor():
    pos = torch.tensor([0, 6, 7, 15, 16])
    t = plain.temperature_factor(pos, 0.1, 8.0, torch.float64)
    assert t[0] == 1.0 and t[1] == 1.0
    assert float(t[2]) == pytest.approx(1 + 0.1 * math.log(2.0))      # floor(8 / 8) = 1
    assert float(t[3]) == pytest.approx(1 + 0.1 * math.log(3.0))
    assert float(t[4]) == pytest.approx(1 + 0.1 * math.log(3.0))


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_model_is_causal_and_chunk_local(model_dirs, name):
    cfg, w = plain.load_folder(model_dirs[name])
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, cfg["vocab_size"], (40,), generator=g).tolist()
    full = plain.forward(cfg, w, toks)
    assert full.shape == (40, cfg["vocab_size"]) and torch.isfinite(full).all()
    assert torch.allclose(plain.forward(cfg, w, toks[:23]), full[:23], atol=1e-9)     # later tokens change nothing
    # float32 agrees with float64 to rounding
    cfg32, w32 = plain.load_folder(model_dirs[name], torch.float32)
    f32 = plain.forward(cfg32, w32, toks)
    assert float((f32.double() - full).abs().max()) < 2e-4 * max(1.0, float(full.abs().max()))


def test_experts_are_really_chosen_per_token(model_dirs):
    cfg, w = plain.load_folder(model_dirs["A"])
    choices = []
    plain.forward(cfg, w, list(range(3, 60)), choices=choices)
    assert len(choices) == 4 and all(len(c) == 57 for c in choices)
    assert len({e for c in choices for e in c}) >= 3


def test_sampling_distribution_filters():
    logits = torch.tensor([2.0, 1.0, 0.5, 0.0, -1.0])
    p = plain.sample_distribution(logits, 1.0)
    assert p.sum() == pytest.approx(1.0) and torch.all(p > 0)
    assert (plain.sample_distribution(logits, 1.0, top_k=2) > 0).tolist() == [True, True, False, False, False]
    assert (plain.sample_distribution(logits, 1.0, min_p=0.3) > 0).tolist() == [True, True, False, False, False]
    keep = plain.sample_distribution(logits, 1.0, top_p=0.7) > 0
    assert keep.tolist() == [True, True, False, False, False]
    assert plain.draw(torch.tensor([0.2, 0.0, 0.5, 0.3]), 0.2) == 0
    assert plain.draw(torch.tensor([0.2, 0.0, 0.5, 0.3]), 0.21) == 2
    assert plain.draw(torch.tensor([0.2, 0.0, 0.5, 0.3]), 0.9999) == 3
