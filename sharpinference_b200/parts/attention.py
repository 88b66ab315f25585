"""Grouped-query attention over the paged cache: the mixer of every Llama 4 layer.

Order of operations for the step's rows (reference: src/SharpInference.Engine/ForwardPass.cs:1576-1690):
fused Q|K|V projection; rotary encoding of q and k; weightless L2 norm of q and k per head
(after the rotation); temperature factor on q; k and v into the request's pages; attention of
every row over the positions its mask lets it see; output projection.  Query head ``h`` reads
kv head ``h // (heads / kv_heads)``; scores are ``q . k / sqrt(d)``.

What the reference lacks is a parameter here: the mask (``full``, ``chunk`` of C positions,
``window`` of W positions), and the temperature factor
``1 + attn_scale * ln(1 + floor((pos + 1) / floor_scale))``.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from ..kernels import ops
from .base import CacheSpec, LayerSlot, Mixer, PositionEncoding, StepContext, register_part
from .linear import Linear
from .norm import L2Norm

_MASK_CODE = {"full": ops.MASK_FULL, "chunk": ops.MASK_CHUNK, "window": ops.MASK_WINDOW}
_PAIRING_CODE = {"interleaved": ops.ROPE_INTERLEAVED, "halves": ops.ROPE_HALVES}


@register_part("mixer", "paged_attention")
class PagedAttention(Mixer):
    def __init__(self, *, qkv: Linear, out: Linear, num_heads: int, num_kv_heads: int, head_dim: int,
                 mask: str = "full", span: int = 0, position: Optional[PositionEncoding] = None,
                 qk_norm: Optional[L2Norm] = None, temperature: Optional[Tuple[float, float]] = None,
                 softmax_scale: Optional[float] = None, act_dtype: torch.dtype = torch.bfloat16):
        if num_heads % num_kv_heads != 0:
            raise ValueError(f"heads ({num_heads}) must be a multiple of kv heads ({num_kv_heads})")
        if head_dim % 2 != 0 or head_dim > 512:
            raise ValueError(f"head size {head_dim} is not supported: it must be even and at most 512")
        if qkv.out_features != (num_heads + 2 * num_kv_heads) * head_dim:
            raise ValueError(f"fused qkv weight has {qkv.out_features} rows, expected "
                             f"(heads + 2 kv_heads) * head_dim = {(num_heads + 2 * num_kv_heads) * head_dim}")
        if out.in_features != num_heads * head_dim:
            raise ValueError(f"output projection reads {out.in_features} columns, expected {num_heads * head_dim}")
        self.qkv, self.out = qkv, out
        self.num_heads, self.num_kv_heads, self.head_dim = num_heads, num_kv_heads, head_dim
        self.cache_spec = CacheSpec(mask, span if mask != "full" else 0, num_kv_heads, head_dim)
        self.position = position
        self.qk_norm = qk_norm
        self.temperature = temperature          # (attn_scale, floor_scale) or None
        self.softmax_scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(head_dim)
        self.act_dtype = act_dtype
        # an encoding that edits q and k itself may look at the step's host-side lists: no graph then
        self.graph_safe = position is None or position.rotary() is not None

    def prefill_tile_rows(self, page_size: int) -> int:
        """Rows of one request that one attention CTA serves in a prompt portion: 128 where the tcgen05
        kernel takes this layer (bfloat16, head size 64 or 128, pages of 64 * 2^k), else 64."""
        return ops.TC_PREFILL_TILE if ops.tc_prefill_supported(self.act_dtype, self.head_dim, page_size) else 64

    def forward(self, ctx: StepContext, slot: LayerSlot, h: torch.Tensor) -> torch.Tensor:
        T = ctx.num_tokens
        nq, nkv, d = self.num_heads, self.num_kv_heads, self.head_dim
        table = ctx.block_tables[slot.group]
        qkv = self.qkv(h)                                                       # [T, (nq + 2 nkv) d] float32

        rot = self.position.rotary() if self.position is not None else None
        if self.position is not None and rot is None and type(self.position).apply is not PositionEncoding.apply:
            # an encoding that is no plain rotation edits q and k itself, before norm and cache write
            q3 = qkv[:, : nq * d].view(T, nq, d)
            k3 = qkv[:, nq * d: (nq + nkv) * d].view(T, nkv, d)
            self.position.apply(ctx, q3, k3)
        inv_freq, pairing = (rot[0], _PAIRING_CODE[rot[1]]) if rot is not None else (None, ops.ROPE_NONE)
        attn_scale, floor_scale = self.temperature if self.temperature is not None else (0.0, 0.0)

        q = torch.empty((T, nq, d), dtype=self.act_dtype, device=h.device)
        ops.qkv_post(qkv, ctx.positions, ctx.row_request, table, inv_freq, q, slot.kv, nq=nq, nkv=nkv, d=d,
                     page_size=slot.page_size, pairing=pairing,
                     l2_eps=self.qk_norm.eps if self.qk_norm is not None else -1.0,
                     temp_attn_scale=attn_scale, temp_floor_scale=floor_scale, write_kv=slot.writes_cache)
        mask_kind, mask_span = _MASK_CODE[self.cache_spec.kind], max(self.cache_spec.span, 1)
        if self.act_dtype == torch.bfloat16 and d in ops.FAST_ATTENTION_HEAD_SIZES and \
                ctx.num_attn_tiles + ctx.num_decode_rows > 0:
            # tensor-core kernels: tiles of prompt rows, and single rows split over their keys
            o = torch.empty((T, nq * d), dtype=torch.bfloat16, device=h.device)
            if ctx.num_attn_tiles:
                prefill = ops.attention_prefill_tc if ctx.attn_tile_rows == ops.TC_PREFILL_TILE else ops.attention_prefill
                prefill(q, slot.kv, table, ctx.attn_tiles, o, nq=nq, nkv=nkv, d=d, page_size=slot.page_size,
                        mask_kind=mask_kind, mask_span=mask_span, scale=self.softmax_scale)
            if ctx.num_decode_rows:
                ops.attention_decode(q, slot.kv, table, ctx.row_request, ctx.positions, o, rows=ctx.decode_rows,
                                     num_rows=ctx.num_decode_rows, nq=nq, nkv=nkv, d=d, page_size=slot.page_size,
                                     mask_kind=mask_kind, mask_span=mask_span, scale=self.softmax_scale,
                                     max_context=ctx.max_context, max_keys=ctx.decode_keys)
        else:
            o = ops.paged_attention_generic(q, slot.kv, table, ctx.row_request, ctx.positions, nq=nq, nkv=nkv, d=d,
                                            page_size=slot.page_size, mask_kind=mask_kind, mask_span=mask_span,
                                            scale=self.softmax_scale)
        return self.out(o)
