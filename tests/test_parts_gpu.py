"""Each part alone against the plain implementation's function for it (needs a GPU)."""
import math
from types import SimpleNamespace

import pytest
import torch

import plain_llama4 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rnd(*shape, scale=1.0, seed=0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def context_for(mixer, lengths_by_step, page_size=8, num_pages=32):
    """A cache manager and step runner around one mixer; yields a StepContext per step."""
    from sharpinference_b200.cache import CacheManager
    from sharpinference_b200.engine.step import StepEntry, StepRunner
    from sharpinference_b200.models.model import ScheduleEntry
    blocks = [SimpleNamespace(mixer=mixer)]
    cache = CacheManager([ScheduleEntry(0)], blocks, page_size=page_size, num_pages=num_pages, max_requests=4,
                         dtype=mixer.act_dtype, device=DEV)
    runner = StepRunner(SimpleNamespace(vocab_size=1 << 30, blocks=blocks), cache)
    return cache, runner, StepEntry


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from sharpinference_b200.parts import RMSNorm
    w = 1 + 0.1 * rnd(120, seed=1)
    x, delta = rnd(9, 120, seed=2), rnd(9, 120, seed=3)
    part = RMSNorm(w.to(DEV), 1e-4)
    xg = x.to(DEV)
    h, h32 = part.apply(xg, delta.to(DEV), rows=None, out_dtype=dtype, want_fp32=True)
    ref = plain.rms_norm((x + delta).double(), w.double(), 1e-4)
    assert torch.allclose(h32.double().cpu(), ref, rtol=1e-5, atol=1e-6)
    assert torch.allclose(h.double().cpu(), ref, rtol=1e-2 if dtype == torch.bfloat16 else 1e-5, atol=1e-3 if dtype == torch.bfloat16 else 1e-6)
    assert torch.allclose(xg.cpu(), x + delta)


@pytest.mark.parametrize("mask,span", [("full", 0), ("chunk", 12), ("window", 7)])
@pytest.mark.parametrize("rope", ["interleaved", "halves", None])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_mixer_alone_in_portions(mask, span, rope, dtype):
    """The mixer over a 50-token sequence cut into portions equals whole-sequence attention."""
    from sharpinference_b200.parts import L2Norm, Linear, PagedAttention, RotaryEncoding, rotary_inv_freq
    H, nq, nkv, d, S = 72, 6, 2, 24, 50
    wq, wk, wv, wo = (rnd(nq * d, H, scale=0.1, seed=4), rnd(nkv * d, H, scale=0.1, seed=5),
                      rnd(nkv * d, H, scale=0.1, seed=6), rnd(H, nq * d, scale=0.1, seed=7))
    if dtype == torch.bfloat16:
        wq, wk, wv, wo = (t.to(torch.bfloat16).float() for t in (wq, wk, wv, wo))
    inv_freq = rotary_inv_freq(d, 5000.0, None)
    mixer = PagedAttention(qkv=Linear(torch.cat([wq, wk, wv]).to(dtype).to(DEV)), out=Linear(wo.to(dtype).to(DEV)),
                           num_heads=nq, num_kv_heads=nkv, head_dim=d, mask=mask, span=span,
                           position=RotaryEncoding(inv_freq.to(DEV), rope) if rope else None,
                           qk_norm=L2Norm(1e-6) if rope else None, temperature=None if rope else (0.3, 4.0),
                           act_dtype=dtype)
    h = rnd(S, H, seed=8)
    if dtype == torch.bfloat16:
        h = h.to(torch.bfloat16).float()
    cache, runner, StepEntry = context_for(mixer, None)
    cache.add_request("a")
    slot = cache.layer_slots()[0]
    outs, at = [], 0
    for n in (7, 2, 13, 1, 1, 26):
        cache.reserve([("a", n)])
        ctx = runner.build_context([StepEntry("a", [0] * n, [])])
        outs.append(mixer.forward(ctx, slot, h[at:at + n].to(dtype).to(DEV)).cpu())
        cache.commit("a", n)
        at += n
    got = torch.cat(outs).double()
    # plain: same formulas on the whole sequence
    hd = h.double()
    pos = torch.arange(S)
    q = (hd @ wq.double().T).reshape(S, nq, d)
    k = (hd @ wk.double().T).reshape(S, nkv, d)
    v = (hd @ wv.double().T).reshape(S, nkv, d)
    if rope == "interleaved":
        q, k = plain.apply_rope(q, pos, inv_freq), plain.apply_rope(k, pos, inv_freq)
    elif rope == "halves":
        def halves(x):
            ang = (pos.float()[:, None] * inv_freq[None, :]).double()
            c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
            a, b = x[..., :d // 2], x[..., d // 2:]
            return torch.cat([a * c - b * s, a * s + b * c], dim=-1)
        q, k = halves(q), halves(k)
    if rope:
        q, k = plain.l2_norm(q, 1e-6), plain.l2_norm(k, 1e-6)
    else:
        q = q * plain.temperature_factor(pos, 0.3, 4.0, torch.float64)[:, None, None]
    ref = plain.attention_scores(q, k, v, plain.visible(mask, span, S)) @ wo.double().T
    scale = float(ref.abs().max())
    err = float((got - ref).abs().max()) / scale
    assert err < (2e-5 if dtype == torch.float32 else 2e-2), err


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dense_feed_forward_part(dtype):
    from sharpinference_b200.parts import DenseSwiGLU, Linear
    H, I, T = 88, 104, 11
    g, u, dn = rnd(I, H, scale=0.1, seed=1), rnd(I, H, scale=0.1, seed=2), rnd(H, I, scale=0.1, seed=3)
    h = rnd(T, H, seed=4)
    if dtype == torch.bfloat16:
        g, u, dn, h = (t.to(torch.bfloat16).float() for t in (g, u, dn, h))
    part = DenseSwiGLU(gate_up=Linear(torch.cat([g, u]).to(dtype).to(DEV)), down=Linear(dn.to(dtype).to(DEV)), act_dtype=dtype)
    out = part.forward(None, h.to(dtype).to(DEV)).double().cpu()
    ref = plain.dense_ffn(h.double(), g.double(), u.double(), dn.double())
    assert float((out - ref).abs().max()) / float(ref.abs().max()) < (1e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_routed_feed_forward_part(dtype):
    from sharpinference_b200.parts import DenseSwiGLU, GroupedLinear, Linear, MoESigmoidTop1
    from sharpinference_b200.parts.base import StepContext
    H, I, E, T = 88, 40, 5, 64
    cfg = {"num_hidden_layers": 1}
    w = {"model.layers.0.feed_forward.router.weight": rnd(E, H, scale=0.3, seed=1),
         "model.layers.0.feed_forward.experts.gate_up_proj": rnd(E, H, 2 * I, scale=0.1, seed=2),
         "model.layers.0.feed_forward.experts.down_proj": rnd(E, I, H, scale=0.1, seed=3),
         "model.layers.0.feed_forward.shared_expert.gate_proj.weight": rnd(I, H, scale=0.1, seed=4),
         "model.layers.0.feed_forward.shared_expert.up_proj.weight": rnd(I, H, scale=0.1, seed=5),
         "model.layers.0.feed_forward.shared_expert.down_proj.weight": rnd(H, I, scale=0.1, seed=6)}
    h = rnd(T, H, seed=7)
    if dtype == torch.bfloat16:
        w = {k: (v if "router" in k else v.to(torch.bfloat16).float()) for k, v in w.items()}
        h = h.to(torch.bfloat16).float()
    p = "model.layers.0.feed_forward."
    shared = DenseSwiGLU(gate_up=Linear(torch.cat([w[p + "shared_expert.gate_proj.weight"], w[p + "shared_expert.up_proj.weight"]]).to(dtype).to(DEV)),
                         down=Linear(w[p + "shared_expert.down_proj.weight"].to(dtype).to(DEV)), act_dtype=dtype)
    part = MoESigmoidTop1(router=w[p + "router.weight"].to(DEV),
                          experts_gate_up=GroupedLinear(w[p + "experts.gate_up_proj"].transpose(1, 2).contiguous().to(dtype).to(DEV)),
                          experts_down=GroupedLinear(w[p + "experts.down_proj"].transpose(1, 2).contiguous().to(dtype).to(DEV)),
                          shared=shared, act_dtype=dtype)
    ctx = SimpleNamespace(extras={"router_choices": []})
    out = part.forward(ctx, h.to(dtype).to(DEV), h.to(DEV)).double().cpu()
    choices = []
    ref = plain.moe_ffn(cfg, {k: v.double() for k, v in w.items()}, 0, h.double(), choices)
    assert ctx.extras["router_choices"][0].cpu().tolist() == choices[0]
    assert len(set(choices[0])) >= 3
    assert float((out - ref).abs().max()) / float(ref.abs().max()) < (1e-5 if dtype == torch.float32 else 1e-2)
    # one row alone gives the same numbers as the row inside the batch
    one = part.forward(SimpleNamespace(extras={}), h[17:18].to(dtype).to(DEV), h[17:18].to(DEV)).double().cpu()
    assert torch.allclose(one, out[17:18], rtol=0, atol=(1e-6 if dtype == torch.float32 else 2e-3) * float(ref.abs().max()))


def test_rotary_part_tables():
    from sharpinference_b200.config.llama4 import RopeScaling
    from sharpinference_b200.parts import RotaryEncoding, rotary_inv_freq
    f = rotary_inv_freq(64, 500000.0, RopeScaling("llama3", 16.0, 1.0, 1.0, 8192))
    base = rotary_inv_freq(64, 500000.0, None)
    wavelen = 2 * math.pi / base
    for j in range(32):
        expect = base[j] / 16.0 if wavelen[j] > 8192 else base[j]
        assert float(f[j]) == pytest.approx(float(expect), rel=1e-6)
    enc = RotaryEncoding(f, "interleaved")
    assert enc.rotary()[1] == "interleaved" and enc.rotary()[0] is f
    with pytest.raises(ValueError):
        RotaryEncoding(f, "diagonal")


def test_unknown_part_kind_names_the_known_ones():
    from sharpinference_b200.parts import make_part, part_kinds
    assert "paged_attention" in part_kinds("mixer") and "moe_sigmoid_top1" in part_kinds("feed_forward")
    with pytest.raises(ValueError, match="paged_attention"):
        make_part("mixer", "telepathy")


def test_linear_on_the_weight_streaming_kernel():
    """The dense products of a decode step run on the weight-streaming kernel, SwiGLU in the gate|up product's
    epilogue; with stream_rows = 0 on the library's, to the same numbers within rounding."""
    from sharpinference_b200.parts import DenseSwiGLU, Linear
    H, I, T = 128, 200, 5
    g, u, dn = rnd(I, H, scale=0.1, seed=1), rnd(I, H, scale=0.1, seed=2), rnd(H, I, scale=0.1, seed=3)
    h = rnd(T, H, seed=4)
    g, u, dn, h = (t.to(torch.bfloat16).float() for t in (g, u, dn, h))
    gate_up = Linear(torch.cat([g, u]).to(torch.bfloat16).to(DEV), stream_rows=64)
    down = Linear(dn.to(torch.bfloat16).to(DEV), stream_rows=64)
    part = DenseSwiGLU(gate_up=gate_up, down=down, act_dtype=torch.bfloat16)
    hb = h.to(torch.bfloat16).to(DEV)
    assert gate_up.streams(hb)
    out = part.forward(None, hb).double().cpu()
    ref = plain.dense_ffn(h.double(), g.double(), u.double(), dn.double())
    assert float((out - ref).abs().max()) / float(ref.abs().max()) < 1e-2
    lib = DenseSwiGLU(gate_up=Linear(gate_up.weight), down=Linear(down.weight), act_dtype=torch.bfloat16)
    assert not lib.gate_up.streams(hb) and not gate_up.streams(rnd(17, H).to(torch.bfloat16).to(DEV))
    assert float((lib.forward(None, hb).double().cpu() - out).abs().max()) / float(ref.abs().max()) < 1e-2


def test_linear_adds_into_its_output():
    """accumulate: the product is added to what the output holds, on the weight-streaming kernel or the grouped
    kernel with K cut over CTAs (both with reductions) and on the library's (product, then an addition); a dense
    SwiGLU passes it on to its down product."""
    from sharpinference_b200.parts import DenseSwiGLU, Linear
    H, I, T = 136, 200, 3
    w = rnd(H, I, scale=0.1, seed=5).to(torch.bfloat16).to(DEV)
    a = rnd(T, I, seed=6).to(torch.bfloat16).to(DEV)
    base = rnd(T, H, seed=7).to(DEV)
    want = base.double().cpu() + a.double().cpu() @ w.double().cpu().T
    for stream_rows, split_add_rows in ((0, 0), (8, 0), (0, 4), (8, 4), (0, 2)):
        lin = Linear(w, stream_rows=stream_rows, split_add_rows=split_add_rows)
        assert lin.streams(a) == (stream_rows > 0)
        assert lin.adds_with_reductions(a) == (stream_rows > 0 or split_add_rows >= T)
        out = base.clone()
        assert lin(a, out=out, accumulate=True) is out
        assert torch.allclose(out.double().cpu(), want, rtol=1e-4, atol=1e-3)
    with pytest.raises(ValueError, match="output"):
        Linear(w)(a, accumulate=True)
    g, u = rnd(I, H, scale=0.1, seed=8).to(torch.bfloat16).to(DEV), rnd(I, H, scale=0.1, seed=9).to(torch.bfloat16).to(DEV)
    h = rnd(T, H, seed=10).to(torch.bfloat16).to(DEV)
    part = DenseSwiGLU(gate_up=Linear(torch.cat([g, u])), down=Linear(w, stream_rows=8), act_dtype=torch.bfloat16)
    alone = part.forward(None, h)
    added = part.forward(None, h, out=base.clone(), accumulate=True)
    assert torch.allclose(added, base + alone, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_linear_with_a_bias(dtype):
    from sharpinference_b200.parts import Linear
    w, b, a = rnd(70, 96, scale=0.1, seed=1), rnd(70, seed=2), rnd(9, 96, seed=3)
    if dtype == torch.bfloat16:
        w, a = w.to(torch.bfloat16).float(), a.to(torch.bfloat16).float()
    want = a.double() @ w.double().T + b.double()
    for stream_rows in (0, 16):
        lin = Linear(w.to(dtype).to(DEV), bias=b.to(DEV), stream_rows=stream_rows)
        # the weight-streaming kernel adds the bias in its epilogue
        assert lin.streams(a.to(dtype).to(DEV)) == (dtype == torch.bfloat16 and stream_rows > 0)
        assert torch.allclose(lin(a.to(dtype).to(DEV)).double().cpu(), want, rtol=1e-4, atol=1e-3)
    with pytest.raises(ValueError, match="bias"):
        Linear(w.to(DEV), bias=b[:5].to(DEV))


def test_l2_norm_is_a_part_of_its_own():
    from sharpinference_b200.parts import L2Norm
    from sharpinference_b200.parts.base import make_part
    x = rnd(17, 48, seed=4)
    part = make_part("norm", "l2", eps=1e-5)
    assert isinstance(part, L2Norm)
    h, h32 = part.apply(x.to(DEV), None, rows=None, out_dtype=torch.bfloat16, want_fp32=True)
    ref = plain.l2_norm(x.double(), 1e-5)
    assert torch.allclose(h32.double().cpu(), ref, rtol=1e-5, atol=1e-6)
    assert torch.allclose(h.double().cpu(), ref, rtol=1e-2, atol=1e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("norm_kind", ["rmsnorm_first", "l2_first", "l2_no_position"])
def test_attention_mixer_with_another_qk_norm(norm_kind, dtype):
    """A weighted norm of q and k before the rotation (and the weightless one in places where it does not fuse
    into the rotation kernel) is a norm part handed to the mixer: nothing in the mixer's kernels changes."""
    from sharpinference_b200.parts import L2Norm, Linear, PagedAttention, RMSNorm, RotaryEncoding, rotary_inv_freq
    H, nq, nkv, d, S = 64, 4, 2, 32, 40
    wq, wk, wv, wo = (rnd(nq * d, H, scale=0.1, seed=4), rnd(nkv * d, H, scale=0.1, seed=5),
                      rnd(nkv * d, H, scale=0.1, seed=6), rnd(H, nq * d, scale=0.1, seed=7))
    if dtype == torch.bfloat16:
        wq, wk, wv, wo = (t.to(torch.bfloat16).float() for t in (wq, wk, wv, wo))
    inv_freq = rotary_inv_freq(d, 5000.0, None)
    nw = 1 + 0.2 * rnd(d, seed=9)
    if norm_kind == "rmsnorm_first":
        norm, first, position = RMSNorm(nw.to(DEV), 1e-5), True, RotaryEncoding(inv_freq.to(DEV), "interleaved")
    elif norm_kind == "l2_first":
        norm, first, position = L2Norm(1e-5), True, RotaryEncoding(inv_freq.to(DEV), "interleaved")
    else:
        norm, first, position = L2Norm(1e-5), False, None
    mixer = PagedAttention(qkv=Linear(torch.cat([wq, wk, wv]).to(dtype).to(DEV)), out=Linear(wo.to(dtype).to(DEV)),
                           num_heads=nq, num_kv_heads=nkv, head_dim=d, mask="full", position=position,
                           qk_norm=norm, qk_norm_first=first, act_dtype=dtype)
    h = rnd(S, H, seed=8)
    if dtype == torch.bfloat16:
        h = h.to(torch.bfloat16).float()
    cache, runner, StepEntry = context_for(mixer, None)
    cache.add_request("a")
    slot = cache.layer_slots()[0]
    outs, at = [], 0
    for n in (11, 1, 1, 20, 7):
        cache.reserve([("a", n)])
        ctx = runner.build_context([StepEntry("a", [0] * n, [])])
        outs.append(mixer.forward(ctx, slot, h[at:at + n].to(dtype).to(DEV)).cpu())
        cache.commit("a", n)
        at += n
    got = torch.cat(outs).double()
    hd, pos = h.double(), torch.arange(S)
    q = (hd @ wq.double().T).reshape(S, nq, d)
    k = (hd @ wk.double().T).reshape(S, nkv, d)
    v = (hd @ wv.double().T).reshape(S, nkv, d)
    if norm_kind == "rmsnorm_first":
        q, k = plain.l2_norm(q, 1e-5) * nw.double(), plain.l2_norm(k, 1e-5) * nw.double()
    else:
        q, k = plain.l2_norm(q, 1e-5), plain.l2_norm(k, 1e-5)
    if position is not None:
        q, k = plain.apply_rope(q, pos, inv_freq), plain.apply_rope(k, pos, inv_freq)
    ref = plain.attention_scores(q, k, v, plain.visible("full", 0, S)) @ wo.double().T
    err = float((got - ref).abs().max()) / float(ref.abs().max())
    assert err < (2e-5 if dtype == torch.float32 else 2e-2), err
    # the one combination that is not built says so
    with pytest.raises(ValueError, match="qk_norm_first"):
        PagedAttention(qkv=mixer.qkv, out=mixer.out, num_heads=nq, num_kv_heads=nkv, head_dim=d,
                       position=RotaryEncoding(inv_freq.to(DEV), "interleaved"), qk_norm=RMSNorm(nw.to(DEV), 1e-5),
                       act_dtype=dtype)
