"""A plain, slow implementation of the Llama 4 text model, for the tests to compare the engine with.

It rests on the formulas of pekkah/SharpInference (each function cites the file and lines it was
written from; paths are relative to the reference project) and, where the reference lacks a
feature of the architecture (chunked attention, the attention-temperature factor, interleaved
dense/mixture layers, the "llama3" rope scaling rule), on the definition written in that
function's docstring.  The reference is C# and cannot be compiled or run on this machine (no
.NET runtime), so no output of its own code is pinned here: this file rests on the formulas.

Whole sequences, no cache, one function per part.  It shares no code with the package: it reads
config.json with ``json`` and the weights with the ``safetensors`` library, and computes in
float64 by default (``dtype=torch.float32`` is available to see what 32-bit rounding alone does).
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch
from safetensors import safe_open


# ---------------------------------------------------------------------------------------
# model folder
# ---------------------------------------------------------------------------------------
def load_folder(model_dir: str, dtype: torch.dtype = torch.float64) -> Tuple[dict, Dict[str, torch.Tensor]]:
    """config.json as a dict and every tensor of model.safetensors, upcast to ``dtype``."""
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as fh:
        cfg = json.load(fh)
    if isinstance(cfg.get("text_config"), dict):
        cfg = cfg["text_config"]
    tensors = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt", device="cpu") as f:
        for name in f.keys():
            key = name[len("language_model."):] if name.startswith("language_model.") else name
            tensors[key] = f.get_tensor(name).to(dtype)
    return cfg, tensors


def nope_layers(cfg: dict) -> List[int]:
    """Layers without rotary encoding.  ``no_rope_layers`` is either a 0/1 flag per layer
    (1 = the layer uses RoPE) or a list of layer numbers; absent: every 4th layer, which is what
    the reference hard-codes (src/SharpInference.Core/ModelGraph.cs:292-295,
    src/SharpInference.Engine/ForwardPass.cs:1617-1618)."""
    L = cfg["num_hidden_layers"]
    v = cfg.get("no_rope_layers")
    if not v:
        return [i for i in range(L) if (i + 1) % 4 == 0]
    if len(v) == L and all(x in (0, 1) for x in v):
        return [i for i, x in enumerate(v) if x == 0]
    return sorted(v)


def moe_layers(cfg: dict) -> List[int]:
    """Layers whose feed-forward is the mixture: an explicit ``moe_layers`` list, else every
    ``interleave_moe_layer_step``-th layer.  (The reference has one global switch,
    src/SharpInference.Core/ModelGraph.cs:264-266.)"""
    if cfg.get("moe_layers") is not None:
        return sorted(cfg["moe_layers"])
    step = cfg.get("interleave_moe_layer_step", 1)
    return [i for i in range(cfg["num_hidden_layers"]) if (i + 1) % step == 0]


# ---------------------------------------------------------------------------------------
# parts
# ---------------------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """``x * 1/sqrt(mean(x^2) + eps) * w`` over the last axis
    (src/SharpInference.Cpu/SimdKernels.cs:4209-4246)."""
    scale = 1.0 / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return x * scale * w


def l2_norm(x: torch.Tensor, eps: float) -> torch.Tensor:
    """The weightless norm of q and k per head: ``x * 1/sqrt(mean(x^2) + eps)``
    (src/SharpInference.Cpu/SimdKernels.cs:4252-4283)."""
    return x * (1.0 / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps))


def rope_frequencies(cfg: dict) -> torch.Tensor:
    """``f_j = 1 / theta^(2j/d)`` in float32 (src/SharpInference.Cpu/SimdKernels.cs:4789-4811),
    then the "llama3" rescaling if configured.  The reference only divides by a stored table
    (src/SharpInference.Engine/ForwardPass.cs:259-276); the rule that makes such a table is:
    with wavelength ``lam = 2 pi / f`` and ``L = original_max_position_embeddings``,
    ``lam < L/high`` keeps f; ``lam > L/low`` gives ``f / factor``; in between
    ``s = (L/lam - low) / (high - low)`` and ``f' = (1 - s) f / factor + s f``."""
    d = cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]
    theta = float(cfg.get("rope_theta", 500000.0))
    f = [1.0 / torch.pow(torch.tensor(theta, dtype=torch.float32),
                         torch.tensor(2.0 * j / d, dtype=torch.float32)) for j in range(d // 2)]
    sc = cfg.get("rope_scaling")
    if sc and sc.get("rope_type", sc.get("type", "llama3")) != "default":
        factor, low, high = float(sc["factor"]), float(sc["low_freq_factor"]), float(sc["high_freq_factor"])
        L = float(sc["original_max_position_embeddings"])
        out = []
        for fj in f:
            ratio = L * fj / (2.0 * math.pi)      # L / lam
            if ratio > high:
                out.append(fj)
            elif ratio < low:
                out.append(fj / factor)
            elif high == low:
                out.append(fj)
            else:
                s = (ratio - low) / (high - low)
                out.append((1.0 - s) * fj / factor + s * fj)
        f = out
    return torch.stack([torch.as_tensor(v, dtype=torch.float32) for v in f])


def apply_rope(x: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """Rotate neighbouring pairs ``(2j, 2j+1)`` of every head by ``pos * f_j``:
    ``(x0, x1) -> (x0 cos a - x1 sin a, x0 sin a + x1 cos a)``
    (src/SharpInference.Cpu/SimdKernels.cs:4591-4629).  ``x`` is [S, heads, d]; the angle is the
    float32 product the reference forms (``angle = p * freqs[i]``, :4805), then upcast."""
    angle = (positions.to(torch.float32)[:, None] * freqs[None, :]).to(x.dtype)   # [S, d/2]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    x0, x1 = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = x0 * cos - x1 * sin
    out[..., 1::2] = x0 * sin + x1 * cos
    return out


def temperature_factor(positions: torch.Tensor, attn_scale: float, floor_scale: float, dtype) -> torch.Tensor:
    """Not in the reference.  ``1 + attn_scale * ln(1 + floor((pos + 1) / floor_scale))`` per
    position, multiplied into q on the layers without rotary encoding."""
    steps = torch.floor((positions.to(torch.float64) + 1.0) / floor_scale)
    return (1.0 + attn_scale * torch.log1p(steps)).to(dtype)


def visible(mask: str, span: int, S: int) -> torch.Tensor:
    """[S, S] boolean: may the query at row p see the key at column t.  The reference is causal
    on every layer (src/SharpInference.Engine/ForwardPass.cs:1850-1851: keys 0 .. pos); a chunked
    layer adds "same chunk of ``span`` positions", a windowed one "within the last ``span``"."""
    p = torch.arange(S)[:, None]
    t = torch.arange(S)[None, :]
    ok = t <= p
    if mask == "chunk":
        ok = ok & (t // span == p // span)
    elif mask == "window":
        ok = ok & (t > p - span)
    return ok


def attention_scores(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, ok: torch.Tensor) -> torch.Tensor:
    """Grouped-query attention of a whole sequence (src/SharpInference.Engine/ForwardPass.cs:1850-1911):
    query head h reads kv head ``h // (heads / kv_heads)``; ``s = q . k / sqrt(d)``; softmax over the
    visible keys; ``o = sum p v``.  q [S, nq, d], k and v [S, nkv, d] -> [S, nq * d]."""
    S, nq, d = q.shape
    nkv = k.shape[1]
    group = nq // nkv
    out = torch.empty(S, nq, d, dtype=q.dtype)
    for h in range(nq):
        kh, vh = k[:, h // group, :], v[:, h // group, :]
        s = (q[:, h, :] @ kh.T) * (1.0 / math.sqrt(d))
        s = s.masked_fill(~ok, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ vh
    return out.reshape(S, nq * d)


def attention_layer(cfg: dict, w: Dict[str, torch.Tensor], i: int, h: torch.Tensor, positions: torch.Tensor,
                    freqs: torch.Tensor, borrowed_kv=None):
    """One attention mixer on normalised activations ``h`` [S, H]: projections without bias
    (src/SharpInference.Engine/ForwardPass.cs:1576-1603); on rotary layers RoPE, then the L2 norm
    of q and k (:1635-1648), a chunk mask; on the others no rotation, no norm, the temperature
    factor on q, a full causal mask; output projection (:1678).  Returns the layer's output and
    its (k, v), which a later layer may borrow instead of computing its own."""
    p = f"model.layers.{i}.self_attn."
    nq, nkv = cfg["num_attention_heads"], cfg.get("num_key_value_heads", cfg["num_attention_heads"])
    d = cfg.get("head_dim") or cfg["hidden_size"] // nq
    S = h.shape[0]
    bias = cfg.get("attention_bias", False)          # a bias where the model stores one (ModelGraph.cs:269-270)
    q = h @ w[p + "q_proj.weight"].T
    k = h @ w[p + "k_proj.weight"].T
    v = h @ w[p + "v_proj.weight"].T
    if bias:
        q, k, v = q + w[p + "q_proj.bias"], k + w[p + "k_proj.bias"], v + w[p + "v_proj.bias"]
    q, k, v = q.reshape(S, nq, d), k.reshape(S, nkv, d), v.reshape(S, nkv, d)
    rope = i not in nope_layers(cfg)
    if rope:
        q, k = apply_rope(q, positions, freqs), apply_rope(k, positions, freqs)
        if cfg.get("use_qk_norm", True):
            # the model's RMSNorm eps unless the file names one (src/SharpInference.Engine/ForwardPass.cs:1642-1648)
            eps = cfg.get("qk_norm_eps", cfg.get("rms_norm_eps", 1e-5))
            q, k = l2_norm(q, eps), l2_norm(k, eps)
        ok = visible("chunk", cfg["attention_chunk_size"], S)
    else:
        if cfg.get("attn_temperature_tuning", True):
            q = q * temperature_factor(positions, cfg.get("attn_scale", 0.1), cfg.get("floor_scale", 8192.0),
                                       q.dtype)[:, None, None]
        ok = visible("full", 0, S)
    if borrowed_kv is not None:
        k, v = borrowed_kv
    o = attention_scores(q, k, v, ok) @ w[p + "o_proj.weight"].T
    if bias:
        o = o + w[p + "o_proj.bias"]
    return o, (k, v)


def silu(x: torch.Tensor) -> torch.Tensor:
    return x / (1.0 + torch.exp(-x))


def dense_ffn(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    """``(silu(h Wg^T) * (h Wu^T)) Wd^T`` (src/SharpInference.Engine/ForwardPass.cs:2006-2015,
    SiLuMul at src/SharpInference.Cpu/SimdKernels.cs:4377-4408)."""
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def moe_ffn(cfg: dict, w: Dict[str, torch.Tensor], i: int, h: torch.Tensor, choices: Optional[list] = None,
            forced: Optional[Sequence[int]] = None, margins: Optional[list] = None):
    """The mixture, token by token as the reference runs it
    (src/SharpInference.Engine/ForwardPass.cs:2021-2098): router logits, sigmoid, the first index
    of the largest value (SelectTopK with k = 1, :2132-2163), the chosen expert's gate and up
    products scaled by the router weight before SiLU (:2082-2088), its down product accumulated
    with weight 1, then the shared expert on the unscaled input added (:2058-2066, :2095-2097).
    Expert tensors: ``gate_up_proj [E, H, 2I]`` multiplies from the right (``h @ W``), its first I
    columns are the gate; ``down_proj [E, I, H]``.

    ``forced`` (one expert per token) replaces the choice, for comparing an implementation whose
    rounding let a near-tie fall the other way: the weight is then the sigmoid of the forced
    expert, and ``margins`` receives, per token, how far below the largest sigmoid the forced
    expert's lies (0 where the choice agrees)."""
    p = f"model.layers.{i}.feed_forward."
    router, gate_up, down = w[p + "router.weight"], w[p + "experts.gate_up_proj"], w[p + "experts.down_proj"]
    I = down.shape[1]
    out = torch.zeros_like(h)
    picked = []
    for t in range(h.shape[0]):
        x = h[t]
        prob = torch.sigmoid(router @ x)
        e, best = 0, prob[0]
        for j in range(1, prob.shape[0]):
            if prob[j] > best:
                e, best = j, prob[j]
        if forced is not None:
            if margins is not None:
                margins.append(float(best - prob[forced[t]]))
            e, best = int(forced[t]), prob[forced[t]]
        picked.append(e)
        gu = x @ gate_up[e]
        g, u = gu[:I] * best, gu[I:] * best
        out[t] = (silu(g) * u) @ down[e]
    if choices is not None:
        choices.append(picked)
    shared = dense_ffn(h, w[p + "shared_expert.gate_proj.weight"], w[p + "shared_expert.up_proj.weight"],
                       w[p + "shared_expert.down_proj.weight"])
    return out + shared


# ---------------------------------------------------------------------------------------
# whole model
# ---------------------------------------------------------------------------------------
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], schedule=None,
            choices: Optional[list] = None, forced: Optional[list] = None,
            margins: Optional[list] = None, layer_norms: Optional[list] = None) -> torch.Tensor:
    """Logits [S, V] of a whole sequence: embedding (src/SharpInference.Engine/ForwardPass.cs:2230-2244),
    then per layer ``x += attn(norm(x))`` and ``x += ffn(norm(x))`` (:1557-1714), the final norm and
    the output product (:1740-1747; the embedding serves as output matrix when tied, :411-413).
    ``schedule`` is a list of ``(layer, borrow)``: run that layer's block, reading the keys and
    values that schedule entry ``borrow`` produced if it is not None; default: every layer once.
    ``forced``: per routed schedule entry, in order, the expert of every token (see ``moe_ffn``).
    ``layer_norms``: a list that receives, per schedule entry, the L2 norm of every position's residual
    after the layer (what SHARPI_TRACE_NORMS prints, :1795-1819)."""
    dtype = w["model.embed_tokens.weight"].dtype
    eps = cfg.get("rms_norm_eps", 1e-5)
    x = w["model.embed_tokens.weight"][torch.as_tensor(list(tokens), dtype=torch.long)]
    positions = torch.arange(len(tokens))
    freqs = rope_frequencies(cfg)
    moe = set(moe_layers(cfg))
    schedule = schedule if schedule is not None else [(i, None) for i in range(cfg["num_hidden_layers"])]
    produced = []
    routed = 0
    for i, borrow in schedule:
        p = f"model.layers.{i}."
        h = rms_norm(x, w[p + "input_layernorm.weight"], eps)
        a, kv = attention_layer(cfg, w, i, h, positions, freqs, None if borrow is None else produced[borrow])
        produced.append(kv)
        x = x + a
        h = rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
        if i in moe:
            m = [] if margins is not None else None
            x = x + moe_ffn(cfg, w, i, h, choices, None if forced is None else forced[routed], m)
            if margins is not None:
                margins.append(m)
            routed += 1
        else:
            x = x + dense_ffn(h, w[p + "feed_forward.gate_proj.weight"], w[p + "feed_forward.up_proj.weight"],
                              w[p + "feed_forward.down_proj.weight"])
        if layer_norms is not None:
            layer_norms.append(x.square().sum(dim=1).sqrt())
    x = rms_norm(x, w["model.norm.weight"], eps)
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return (x @ head.T).to(dtype)


def greedy(logits: torch.Tensor) -> int:
    """Left to right, strict ``>``: the lowest index wins a tie
    (src/SharpInference.Engine/Sampler.cs:436-449)."""
    best, idx = logits[0], 0
    for i in range(1, logits.shape[0]):
        if logits[i] > best:
            best, idx = logits[i], i
    return idx


def generate_greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], n: int) -> List[int]:
    """Prefill, pick, append, run the whole sequence again (no cache): the decode loop of
    src/SharpInference.Cli/RunCommand.cs:2256-2291 with ``Greedy``."""
    seq = list(prompt)
    out = []
    for _ in range(n):
        tok = greedy(forward(cfg, w, seq)[-1])
        out.append(tok)
        seq.append(tok)
    return out


def sample_distribution(logits: torch.Tensor, temperature: float, top_k: int = 0, top_p: float = 1.0,
                        min_p: float = 0.0) -> torch.Tensor:
    """The distribution the reference draws from (src/SharpInference.Engine/Sampler.cs:71-107):
    logits / T, softmax, keep the top-k (ties at the k-th value stay) and renormalise, drop below
    ``min_p * max``, keep the smallest most-probable set whose mass reaches top_p, renormalise."""
    p = torch.softmax(logits.to(torch.float64) / temperature, dim=-1)
    if 0 < top_k < p.shape[0]:
        kth = torch.sort(p, descending=True).values[top_k - 1]
        p = torch.where(p < kth, torch.zeros_like(p), p)
        p = p / p.sum()
    if min_p > 0:
        p = torch.where(p < min_p * p.max(), torch.zeros_like(p), p)
    if 0 < top_p < 1:
        order = torch.argsort(p, descending=True)
        csum = torch.cumsum(p[order], dim=0)
        reached = (csum >= top_p).nonzero()
        cut = int(reached[0].item()) + 1 if reached.numel() else p.shape[0]      # never reached: everything stays
        keep = torch.zeros_like(p)
        keep[order[:cut]] = p[order[:cut]]
        p = keep
    return p / p.sum()


def draw(p: torch.Tensor, u: float) -> int:
    """First index whose cumulative probability reaches ``u``
    (src/SharpInference.Engine/Sampler.cs:564-576)."""
    c = 0.0
    last = 0
    for i in range(p.shape[0]):
        if p[i] > 0:
            last = i
        c += float(p[i])
        if u <= c and p[i] > 0:
            return i
    return last
