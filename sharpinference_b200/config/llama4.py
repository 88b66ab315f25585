"""``Llama4TextConfig``: the typed configuration of the Llama 4 text architecture.

Every size and constant of the model comes from the keys that a Llama 4 ``config.json``
itself carries (at the top level, or inside its ``text_config`` member for a multimodal
checkpoint).  The reference reads the same quantities from model metadata into one typed
record (src/SharpInference.Core/ModelGraph.cs:492-543) and hard-codes what the metadata
lacks, e.g. "every 4th layer has no RoPE" (src/SharpInference.Core/ModelGraph.cs:292-295);
here those are data: ``no_rope_layers``, ``interleave_moe_layer_step`` / ``moe_layers``.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ConfigError, ConfigReader


@dataclass(frozen=True)
class RopeScaling:
    """Frequency-dependent "llama3" scaling of the rotary frequencies."""

    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int


@dataclass(frozen=True)
class Llama4TextConfig:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int          # width of one routed expert and of the shared expert
    intermediate_size_mlp: int      # width of the dense feed-forward on non-MoE layers
    num_local_experts: int
    num_experts_per_tok: int
    moe_layers: Tuple[int, ...]     # indices of the layers whose feed-forward is MoE
    rope_theta: float
    rope_scaling: Optional[RopeScaling]
    no_rope_layers: Tuple[int, ...]  # indices of the layers WITHOUT rotary encoding (global attention)
    attention_chunk_size: int
    use_qk_norm: bool
    qk_norm_eps: float
    attn_temperature_tuning: bool
    floor_scale: float
    attn_scale: float
    rms_norm_eps: float
    tie_word_embeddings: bool
    max_position_embeddings: int
    eos_token_ids: Tuple[int, ...]
    bos_token_id: Optional[int]
    interleave_moe_layer_step: int
    attention_bias: bool = False        # q, k, v and o projections carry a bias vector

    architecture = "Llama4ForCausalLM"

    # -- per-layer questions -----------------------------------------------------------
    def layer_uses_rope(self, layer: int) -> bool:
        return layer not in self.no_rope_layers

    def layer_is_moe(self, layer: int) -> bool:
        return layer in self.moe_layers

    # -- reading -----------------------------------------------------------------------
    @classmethod
    def from_dict(cls, obj: dict, where: str = "config.json") -> "Llama4TextConfig":
        top = obj
        if isinstance(obj.get("text_config"), dict):
            obj = obj["text_config"]
            where = f"{where}[text_config]"
        r = ConfigReader(obj, where)

        vocab = r.int("vocab_size")
        hidden = r.int("hidden_size")
        layers = r.int("num_hidden_layers")
        heads = r.int("num_attention_heads")
        kv_heads = r.int("num_key_value_heads", heads)
        head_dim = r.int("head_dim", (hidden // heads) if (hidden and heads) else None)
        inter = r.int("intermediate_size")
        inter_mlp = r.int("intermediate_size_mlp", inter)
        experts = r.int("num_local_experts")
        per_tok = r.int("num_experts_per_tok", 1)
        step = r.int("interleave_moe_layer_step", 1)
        moe_layers = r.int_list("moe_layers", None)
        theta = r.float("rope_theta", 500000.0)
        scaling_obj = r.object("rope_scaling", None)
        no_rope = r.int_list("no_rope_layers", None)
        chunk = r.int("attention_chunk_size")
        qk_norm = r.bool("use_qk_norm", True)
        eps = r.float("rms_norm_eps", 1e-5)
        # The weightless q/k norm takes the model's RMSNorm eps (src/SharpInference.Engine/ForwardPass.cs:1642-1648
        # passes _hp.RmsNormEps); checkpoints carry no key of its own.  An explicit `qk_norm_eps` overrides it.
        qk_eps = r.float("qk_norm_eps", eps)
        temp_tuning = r.switch("attn_temperature_tuning", True)
        floor_scale = r.float("floor_scale", 8192.0)
        attn_scale = r.float("attn_scale", 0.1)
        nope_interval = r.int("no_rope_layer_interval", 4)
        tied = r.bool("tie_word_embeddings", bool(top.get("tie_word_embeddings", False)))
        max_pos = r.int("max_position_embeddings", 1 << 20)
        act = r.str("hidden_act", "silu")
        attn_bias = r.bool("attention_bias", False)
        bos = r.int("bos_token_id", None)

        eos_raw = obj.get("eos_token_id", None)
        eos: Tuple[int, ...] = ()
        if isinstance(eos_raw, int) and not isinstance(eos_raw, bool):
            eos = (eos_raw,)
        elif isinstance(eos_raw, list) and all(isinstance(v, int) and not isinstance(v, bool) for v in eos_raw):
            eos = tuple(eos_raw)
        elif eos_raw is not None:
            r.problem(f"key 'eos_token_id': expected an integer or a list of integers, found {eos_raw!r}")

        scaling = None
        if scaling_obj is not None:
            s = ConfigReader(scaling_obj, f"{where}[rope_scaling]")
            rope_type = s.str("rope_type", scaling_obj.get("type", None) if isinstance(scaling_obj.get("type"), str) else "llama3")
            if rope_type == "default":
                scaling = None
            elif rope_type != "llama3":
                r.problem(f"rope_scaling.rope_type '{rope_type}' is not supported (known: 'llama3', 'default')")
            else:
                scaling = RopeScaling(
                    rope_type=rope_type,
                    factor=s.float("factor"),
                    low_freq_factor=s.float("low_freq_factor"),
                    high_freq_factor=s.float("high_freq_factor"),
                    original_max_position_embeddings=s.int("original_max_position_embeddings"),
                )
                try:
                    s.finish()
                except ConfigError as exc:
                    r.problem(str(exc))
                    scaling = None

        if not r.ok:
            r.finish()

        # ---- derived lists -----------------------------------------------------------
        if moe_layers is None:
            r.require(step >= 1, f"interleave_moe_layer_step must be >= 1, found {step}")
            moe = tuple(i for i in range(layers) if step >= 1 and (i + 1) % step == 0)
        else:
            moe = tuple(sorted(set(moe_layers)))
            r.require(all(0 <= i < layers for i in moe), f"moe_layers {moe_layers} holds an index outside [0, {layers})")

        r.require(nope_interval is not None and nope_interval >= 1,
                  f"no_rope_layer_interval must be >= 1, found {nope_interval}")
        nope = _parse_no_rope_layers(no_rope, layers, r, nope_interval or 4)

        # ---- validation --------------------------------------------------------------
        for name, value in (("vocab_size", vocab), ("hidden_size", hidden), ("num_hidden_layers", layers),
                            ("num_attention_heads", heads), ("num_key_value_heads", kv_heads),
                            ("head_dim", head_dim), ("intermediate_size", inter),
                            ("intermediate_size_mlp", inter_mlp), ("attention_chunk_size", chunk),
                            ("max_position_embeddings", max_pos)):
            r.require(value is not None and value > 0, f"{name} must be positive, found {value}")
        if heads and kv_heads and heads > 0 and kv_heads > 0:
            r.require(heads % kv_heads == 0,
                      f"num_attention_heads ({heads}) must be a multiple of num_key_value_heads ({kv_heads})")
        if head_dim:
            r.require(head_dim % 2 == 0, f"head_dim must be even for rotary pairs, found {head_dim}")
        if moe:
            r.require(experts >= 1, f"num_local_experts must be >= 1 when there are MoE layers, found {experts}")
        r.require(per_tok == 1, f"num_experts_per_tok must be 1 (top-1 sigmoid router), found {per_tok}")
        r.require(act == "silu", f"hidden_act must be 'silu', found '{act}'")
        r.require(eps is not None and qk_eps is not None and eps > 0 and qk_eps > 0,
                  "rms_norm_eps and qk_norm_eps must be positive")
        r.require(theta > 0, f"rope_theta must be positive, found {theta}")
        if temp_tuning:
            r.require(floor_scale > 0, f"floor_scale must be positive, found {floor_scale}")
        if scaling is not None:
            r.require(scaling.factor > 0, "rope_scaling.factor must be positive")
            r.require(scaling.original_max_position_embeddings > 0,
                      "rope_scaling.original_max_position_embeddings must be positive")
            r.require(scaling.high_freq_factor >= scaling.low_freq_factor,
                      "rope_scaling.high_freq_factor must be >= low_freq_factor")
        r.finish()

        return cls(
            vocab_size=vocab, hidden_size=hidden, num_hidden_layers=layers, num_attention_heads=heads,
            num_key_value_heads=kv_heads, head_dim=head_dim, intermediate_size=inter,
            intermediate_size_mlp=inter_mlp, num_local_experts=experts, num_experts_per_tok=per_tok,
            moe_layers=moe, rope_theta=theta, rope_scaling=scaling, no_rope_layers=nope,
            attention_chunk_size=chunk, use_qk_norm=qk_norm, qk_norm_eps=qk_eps,
            attn_temperature_tuning=temp_tuning, floor_scale=floor_scale, attn_scale=attn_scale,
            rms_norm_eps=eps, tie_word_embeddings=tied, max_position_embeddings=max_pos,
            eos_token_ids=eos, bos_token_id=bos, interleave_moe_layer_step=step,
            attention_bias=bool(attn_bias),
        )

    # -- writing -----------------------------------------------------------------------
    def to_dict(self) -> dict:
        """A ``config.json`` object that ``from_dict`` reads back to an equal configuration."""
        out = {
            "architectures": [self.architecture],
            "model_type": "llama4_text",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "intermediate_size_mlp": self.intermediate_size_mlp,
            "num_local_experts": self.num_local_experts,
            "num_experts_per_tok": self.num_experts_per_tok,
            "interleave_moe_layer_step": self.interleave_moe_layer_step,
            "moe_layers": list(self.moe_layers),
            "rope_theta": self.rope_theta,
            "rope_scaling": None if self.rope_scaling is None else dataclasses.asdict(self.rope_scaling),
            "no_rope_layers": [int(self.layer_uses_rope(i)) for i in range(self.num_hidden_layers)],
            "attention_chunk_size": self.attention_chunk_size,
            "use_qk_norm": self.use_qk_norm,
            "qk_norm_eps": self.qk_norm_eps,
            "attn_temperature_tuning": self.attn_temperature_tuning,
            # whole numbers are written as integers, which is the form checkpoints carry
            "floor_scale": int(self.floor_scale) if float(self.floor_scale).is_integer() else self.floor_scale,
            "attn_scale": self.attn_scale,
            "rms_norm_eps": self.rms_norm_eps,
            "tie_word_embeddings": self.tie_word_embeddings,
            "max_position_embeddings": self.max_position_embeddings,
            "hidden_act": "silu",
            "attention_bias": self.attention_bias,
        }
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        return out


def _parse_no_rope_layers(value: Optional[list], layers: int, r: ConfigReader, interval: int = 4) -> Tuple[int, ...]:
    """``no_rope_layers`` is written in two ways; both mean "which layers skip RoPE".

    * per-layer flags: a list of length ``num_hidden_layers`` of 0/1, where **1 means the
      layer uses RoPE** and 0 means it does not (the form checkpoints carry);
    * indices: a list of the layer numbers without RoPE, e.g. ``[3]`` or ``[2, 5]``.

    A list is read as flags exactly when its length equals ``num_hidden_layers`` and every
    entry is 0 or 1; otherwise as indices.  Absent or empty: the architecture's rule, every
    ``interval``-th layer (``(i + 1) % interval == 0``; ``no_rope_layer_interval``, 4 when the
    file does not say) is without RoPE; the reference fixes 4 in code
    (src/SharpInference.Core/ModelGraph.cs:292-295).
    """
    if not layers or layers <= 0:
        return ()
    if value is None or len(value) == 0:
        return tuple(i for i in range(layers) if (i + 1) % max(interval, 1) == 0)
    if len(value) == layers and all(v in (0, 1) for v in value):
        return tuple(i for i, v in enumerate(value) if v == 0)
    idx = tuple(sorted(set(value)))
    r.require(all(0 <= i < layers for i in idx), f"no_rope_layers {value} holds an index outside [0, {layers})")
    r.require(len(idx) == len(value), f"no_rope_layers {value} names a layer twice")
    return idx
