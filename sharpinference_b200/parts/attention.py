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
from typing import Hashable, Optional, Sequence, Tuple

import numpy as np
import torch

from ..kernels import ops
from .base import (CacheSpec, LayerSlot, Mixer, Norm, PositionEncoding, StepContext, StepPlanData, StepPlanner,
                   register_part)
from .linear import Linear

_MASK_CODE = {"full": ops.MASK_FULL, "chunk": ops.MASK_CHUNK, "window": ops.MASK_WINDOW}
_PAIRING_CODE = {"interleaved": ops.ROPE_INTERLEAVED, "halves": ops.ROPE_HALVES}


class PagedAttentionPlanner(StepPlanner):
    """How the attention kernels split a step's rows: portions of prompts become tiles of up to ``tile_rows``
    consecutive rows of one request (int32 ``tiles`` [n, 4]: first row, rows, first position, request index),
    which the prompt kernels serve one CTA (per head) each; entries of up to ``DECODE_ROWS_UP_TO`` rows are
    served row by row by the split-KV kernel (int32 ``decode_rows`` [m]; left out when every row of the step
    is such a row).  ``decode_keys`` bounds the sum of position + 1 over the single rows: the split-KV launch
    holds about as many CTAs as these rows have 256-key splits together."""

    DECODE_ROWS_UP_TO = 4

    def __init__(self, tile_rows: int):
        self.tile_rows = int(tile_rows)
        self.key = ("paged_attention", self.tile_rows)

    @staticmethod
    def keys_bucket(keys: int, rows: int = 1) -> int:
        """``keys`` rounded up to a multiple of a power of two: a sixteenth to an eighth of ``keys``, and at
        least 256 keys a row, so that a batch that gains a key a row each step stays in its bucket for 256
        steps or more (a new bucket means a step run eagerly and a graph captured)."""
        step = 1 << max((256 * max(rows, 1) - 1).bit_length(), keys.bit_length() - 4)
        return (keys + step - 1) // step * step

    def bucket(self, starts: Sequence[int], lengths: Sequence[int]) -> Hashable:
        return self.keys_bucket(sum(s + 1 for s in starts), len(starts))

    def plan(self, starts: Sequence[int], lengths: Sequence[int], bucket: Hashable = None) -> StepPlanData:
        tiles, decode_rows = [], []
        keys = 0                         # sum of position + 1 over the single rows
        r = 0
        for b, (start, n) in enumerate(zip(starts, lengths)):
            if n <= self.DECODE_ROWS_UP_TO:
                decode_rows.extend(range(r, r + n))
                keys += n * start + n * (n + 1) // 2
            else:
                for t0 in range(0, n, self.tile_rows):
                    tiles.append((r + t0, min(self.tile_rows, n - t0), start + t0, b))
            r += n
        all_single = len(decode_rows) == r
        return StepPlanData(
            arrays={"tiles": np.asarray(tiles, dtype=np.int32).reshape(-1, 4),
                    "decode_rows": np.asarray([] if all_single else decode_rows, dtype=np.int32)},
            values={"num_tiles": len(tiles), "num_decode_rows": len(decode_rows), "tile_rows": self.tile_rows,
                    "decode_keys": keys if bucket is None else int(bucket)})


@register_part("mixer", "paged_attention")
class PagedAttention(Mixer):
    def __init__(self, *, qkv: Linear, out: Linear, num_heads: int, num_kv_heads: int, head_dim: int,
                 mask: str = "full", span: int = 0, position: Optional[PositionEncoding] = None,
                 qk_norm: Optional[Norm] = None, qk_norm_first: bool = False,
                 temperature: Optional[Tuple[float, float]] = None,
                 softmax_scale: Optional[float] = None, act_dtype: torch.dtype = torch.bfloat16):
        """``qk_norm``: any :class:`Norm` over the head size, applied to every head of q and k; after the
        position encoding (Llama 4's order) unless ``qk_norm_first``.  The weightless L2 norm after a rotation
        runs inside the kernel that rotates and writes the cache; every other combination applies the norm as
        a launch of its own on q and on k."""
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
        self.qk_norm_first = bool(qk_norm_first)
        rotary = position is not None and position.rotary() is not None
        # the fused kernel's order is rotation, weightless norm, temperature
        self._norm_fused = (qk_norm is not None and not qk_norm_first
                            and getattr(qk_norm, "fuses_into_rotation", False))
        if qk_norm is not None and not self._norm_fused and not qk_norm_first and rotary:
            raise ValueError(f"a q/k norm of kind '{qk_norm.kind}' after a rotary encoding is not built (only the "
                             f"weightless L2 norm fuses into the rotation kernel): place it before the position "
                             f"encoding (qk_norm_first=True) or use an encoding that edits q and k itself")
        self.temperature = temperature          # (attn_scale, floor_scale) or None
        self.softmax_scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(head_dim)
        self.act_dtype = act_dtype
        # an encoding that edits q and k itself may look at the step's host-side lists: no graph then
        self.graph_safe = position is None or position.rotary() is not None

    def prefill_tile_rows(self, page_size: int) -> int:
        """Rows of one request that one attention CTA serves in a prompt portion: 128 where the tcgen05
        kernel takes this layer (bfloat16, head size 64 or 128, pages of 64 * 2^k), else 64."""
        return ops.TC_PREFILL_TILE if ops.tc_prefill_supported(self.act_dtype, self.head_dim, page_size) else 64

    def step_planner(self, page_size: int) -> StepPlanner:
        return PagedAttentionPlanner(self.prefill_tile_rows(page_size))

    def _norm_heads(self, qkv: torch.Tensor, T: int) -> None:
        """The q/k norm as a part of its own: every head of q and of k is a row of width head_dim."""
        nq, nkv, d = self.num_heads, self.num_kv_heads, self.head_dim
        for first, heads in ((0, nq), (nq * d, nkv)):
            cols = qkv[:, first:first + heads * d]
            rows = cols.reshape(T * heads, d).contiguous()
            normed, _ = self.qk_norm.apply(rows, None, rows=None, out_dtype=torch.float32)
            cols.copy_(normed.view(T, heads * d))

    def forward(self, ctx: StepContext, slot: LayerSlot, h: torch.Tensor) -> torch.Tensor:
        T = ctx.num_tokens
        plan = ctx.plans[("paged_attention", self.prefill_tile_rows(slot.page_size))]
        nq, nkv, d = self.num_heads, self.num_kv_heads, self.head_dim
        table = ctx.block_tables[slot.group]
        qkv = self.qkv(h)                                                       # [T, (nq + 2 nkv) d] float32

        rot = self.position.rotary() if self.position is not None else None
        if self.position is not None and rot is None and type(self.position).apply is not PositionEncoding.apply:
            # an encoding that is no plain rotation edits q and k itself, before norm and cache write
            q3 = qkv[:, : nq * d].view(T, nq, d)
            k3 = qkv[:, nq * d: (nq + nkv) * d].view(T, nkv, d)
            if self.qk_norm is not None and self.qk_norm_first:
                self._norm_heads(qkv, T)
            self.position.apply(ctx, q3, k3)
            if self.qk_norm is not None and not self.qk_norm_first and not self._norm_fused:
                self._norm_heads(qkv, T)
        elif self.qk_norm is not None and not self._norm_fused:
            self._norm_heads(qkv, T)             # before a rotation, or with no position encoding at all
        inv_freq, pairing = (rot[0], _PAIRING_CODE[rot[1]]) if rot is not None else (None, ops.ROPE_NONE)
        attn_scale, floor_scale = self.temperature if self.temperature is not None else (0.0, 0.0)

        q = torch.empty((T, nq, d), dtype=self.act_dtype, device=h.device)
        ops.qkv_post(qkv, ctx.positions, ctx.row_request, table, inv_freq, q, slot.kv, nq=nq, nkv=nkv, d=d,
                     page_size=slot.page_size, pairing=pairing,
                     l2_eps=self.qk_norm.eps if self._norm_fused else -1.0,
                     temp_attn_scale=attn_scale, temp_floor_scale=floor_scale, write_kv=slot.writes_cache)
        mask_kind, mask_span = _MASK_CODE[self.cache_spec.kind], max(self.cache_spec.span, 1)
        if self.act_dtype == torch.bfloat16 and d in ops.FAST_ATTENTION_HEAD_SIZES:
            # tensor-core kernels: tiles of prompt rows, and single rows split over their keys
            o = torch.empty((T, nq * d), dtype=torch.bfloat16, device=h.device)
            if plan.num_tiles:
                prefill = ops.attention_prefill_tc if plan.tile_rows == ops.TC_PREFILL_TILE else ops.attention_prefill
                prefill(q, slot.kv, table, plan.tiles, o, nq=nq, nkv=nkv, d=d, page_size=slot.page_size,
                        mask_kind=mask_kind, mask_span=mask_span, scale=self.softmax_scale)
            if plan.num_decode_rows:
                ops.attention_decode(q, slot.kv, table, ctx.row_request, ctx.positions, o, rows=plan.decode_rows,
                                     num_rows=plan.num_decode_rows, nq=nq, nkv=nkv, d=d, page_size=slot.page_size,
                                     mask_kind=mask_kind, mask_span=mask_span, scale=self.softmax_scale,
                                     max_context=ctx.max_context, max_keys=plan.decode_keys)
        else:
            o = ops.paged_attention_generic(q, slot.kv, table, ctx.row_request, ctx.positions, nq=nq, nkv=nkv, d=d,
                                            page_size=slot.page_size, mask_kind=mask_kind, mask_span=mask_span,
                                            scale=self.softmax_scale)
        return self.out(o)
