"""The Llama 4 text architecture, put together from parts, and its tensor names.

Per layer (constants from :class:`Llama4TextConfig`):

* mixer: grouped-query attention; on rotary layers a chunk mask of ``attention_chunk_size``
  positions, interleaved-pair rotation (with "llama3" frequency scaling if configured) and, if
  ``use_qk_norm``, the weightless L2 norm of q and k after the rotation; on the layers listed in
  ``no_rope_layers`` a full causal mask, no rotation, no norm, and the temperature factor on q if
  ``attn_temperature_tuning``.
* feed-forward: a top-1 sigmoid-routed mixture with a shared expert on ``moe_layers``, a dense
  SwiGLU of width ``intermediate_size_mlp`` elsewhere.

The reference reads the same model from GGUF tensor names
(src/SharpInference.Engine/ForwardPass.cs:289-413).  The names below are those of the
architecture's safetensors checkpoints: per-layer ``self_attn.{q,k,v,o}_proj.weight``,
``input_layernorm.weight``, ``post_attention_layernorm.weight``; mixture layers
``feed_forward.router.weight [E, H]``, ``feed_forward.experts.gate_up_proj [E, H, 2I]`` (input-major:
``x @ W``; the first I columns are the gate, the last I the up projection),
``feed_forward.experts.down_proj [E, I, H]`` (or, where a folder keeps the experts apart,
``feed_forward.experts.<e>.{gate,up,down}_proj.weight`` as ``[out, in]`` matrices),
``feed_forward.shared_expert.{gate,up,down}_proj.weight``;
dense layers ``feed_forward.{gate,up,down}_proj.weight``; ``model.embed_tokens.weight``,
``model.norm.weight``, ``lm_head.weight``; with ``attention_bias`` also ``self_attn.{q,k,v,o}_proj.bias``
(the reference probes for a bias tensor, src/SharpInference.Core/ModelGraph.cs:269-270).  Q, K and V are
concatenated for one product, gate and up likewise, and the expert tensors are transposed once to
``[E, out, in]``.
"""
from __future__ import annotations

import torch

from ..config.llama4 import Llama4TextConfig
from ..parts import (DenseSwiGLU, GroupedLinear, L2Norm, Linear, MoESigmoidTop1, PagedAttention, PreNormBlock,
                     RMSNorm, RotaryEncoding, rotary_inv_freq)
from ..registry import register_architecture
from ..weights.source import WeightSource
from .model import DecoderModel


def _cat(tensors, dim=0):
    dtypes = {t.dtype for t in tensors}
    if len(dtypes) > 1:   # one of them was stored in 32-bit: the fused product is 32-bit
        tensors = [t.to(torch.float32) for t in tensors]
    return torch.cat(tensors, dim=dim).contiguous()


def build_llama4(config: Llama4TextConfig, weights: WeightSource) -> DecoderModel:
    c = config
    act = weights.compute_dtype
    H, d, nq, nkv = c.hidden_size, c.head_dim, c.num_attention_heads, c.num_key_value_heads

    embedding = weights.matrix("model.embed_tokens.weight", (c.vocab_size, H))
    inv_freq = rotary_inv_freq(d, c.rope_theta, c.rope_scaling)
    if weights.device.type != "meta":
        inv_freq = inv_freq.to(weights.device)
    rotary = RotaryEncoding(inv_freq, "interleaved")

    blocks = []
    for i in range(c.num_hidden_layers):
        p = f"model.layers.{i}."
        qkv = _cat([weights.matrix(p + "self_attn.q_proj.weight", (nq * d, H)),
                    weights.matrix(p + "self_attn.k_proj.weight", (nkv * d, H)),
                    weights.matrix(p + "self_attn.v_proj.weight", (nkv * d, H))])
        o = weights.matrix(p + "self_attn.o_proj.weight", (H, nq * d))
        qkv_bias = o_bias = None
        if c.attention_bias:
            qkv_bias = torch.cat([weights.vector(p + "self_attn.q_proj.bias", (nq * d,), init="normal"),
                                  weights.vector(p + "self_attn.k_proj.bias", (nkv * d,), init="normal"),
                                  weights.vector(p + "self_attn.v_proj.bias", (nkv * d,), init="normal")]).contiguous()
            o_bias = weights.vector(p + "self_attn.o_proj.bias", (H,), init="normal")
        if c.layer_uses_rope(i):
            mixer = PagedAttention(qkv=Linear(qkv, p + "qkv", bias=qkv_bias), out=Linear(o, p + "o", bias=o_bias), num_heads=nq,
                                   num_kv_heads=nkv, head_dim=d, mask="chunk", span=c.attention_chunk_size,
                                   position=rotary, qk_norm=L2Norm(c.qk_norm_eps) if c.use_qk_norm else None,
                                   temperature=None, act_dtype=act)
        else:
            mixer = PagedAttention(qkv=Linear(qkv, p + "qkv", bias=qkv_bias), out=Linear(o, p + "o", bias=o_bias),
                                   num_heads=nq, num_kv_heads=nkv, head_dim=d, mask="full", position=None, qk_norm=None,
                                   temperature=(c.attn_scale, c.floor_scale) if c.attn_temperature_tuning else None,
                                   act_dtype=act)
        if c.layer_is_moe(i):
            E, I = c.num_local_experts, c.intermediate_size
            router = weights.vector(p + "feed_forward.router.weight", (E, H), init="normal")
            if weights.stored(p + "feed_forward.experts.0.gate_proj.weight"):
                # one set of [out, in] matrices per expert
                e_gate_up = torch.stack([_cat([weights.matrix(f"{p}feed_forward.experts.{e}.gate_proj.weight", (I, H)),
                                               weights.matrix(f"{p}feed_forward.experts.{e}.up_proj.weight", (I, H))])
                                         for e in range(E)])
                e_down = torch.stack([weights.matrix(f"{p}feed_forward.experts.{e}.down_proj.weight", (H, I))
                                      for e in range(E)])
            else:
                # the fused, input-major tensors
                e_gate_up = weights.matrix(p + "feed_forward.experts.gate_up_proj", (E, H, 2 * I)).transpose(1, 2).contiguous()
                e_down = weights.matrix(p + "feed_forward.experts.down_proj", (E, I, H)).transpose(1, 2).contiguous()
            shared = DenseSwiGLU(
                gate_up=Linear(_cat([weights.matrix(p + "feed_forward.shared_expert.gate_proj.weight", (I, H)),
                                     weights.matrix(p + "feed_forward.shared_expert.up_proj.weight", (I, H))]),
                               p + "shared.gate_up"),
                down=Linear(weights.matrix(p + "feed_forward.shared_expert.down_proj.weight", (H, I)), p + "shared.down"),
                act_dtype=act)
            ffn = MoESigmoidTop1(router=router,
                                 experts_gate_up=GroupedLinear(e_gate_up, p + "experts.gate_up"),
                                 experts_down=GroupedLinear(e_down, p + "experts.down"),
                                 shared=shared, act_dtype=act)
        else:
            I = c.intermediate_size_mlp
            ffn = DenseSwiGLU(
                gate_up=Linear(_cat([weights.matrix(p + "feed_forward.gate_proj.weight", (I, H)),
                                     weights.matrix(p + "feed_forward.up_proj.weight", (I, H))]), p + "gate_up"),
                down=Linear(weights.matrix(p + "feed_forward.down_proj.weight", (H, I)), p + "down"), act_dtype=act)
        blocks.append(PreNormBlock(
            mixer_norm=RMSNorm(weights.vector(p + "input_layernorm.weight", (H,)), c.rms_norm_eps), mixer=mixer,
            ffn_norm=RMSNorm(weights.vector(p + "post_attention_layernorm.weight", (H,)), c.rms_norm_eps), ffn=ffn,
            act_dtype=act))

    final_norm = RMSNorm(weights.vector("model.norm.weight", (H,)), c.rms_norm_eps)
    head_weight = embedding if c.tie_word_embeddings else weights.matrix("lm_head.weight", (c.vocab_size, H))
    return DecoderModel(embedding=embedding, blocks=blocks, final_norm=final_norm,
                        head=Linear(head_weight, "lm_head"), act_dtype=act, eos_token_ids=c.eos_token_ids, config=c)


register_architecture("Llama4ForCausalLM", Llama4TextConfig, build_llama4,
                      aliases=("Llama4ForConditionalGeneration",))
