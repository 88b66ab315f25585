"""The arrangement of a layer's parts around the residual stream.

``PreNormBlock`` is the reference's order (src/SharpInference.Engine/ForwardPass.cs:1557-1714):
``x += mixer(norm1(x))``, then ``x += ffn(norm2(x))``.  The residual stream is float32; each
residual add is fused into the norm that follows it, so a block returns its feed-forward output
as ``pending`` and the next block's first norm (or the model's last) adds it.
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import Block, FeedForward, LayerSlot, Mixer, Norm, StepContext, register_part


@register_part("block", "prenorm")
class PreNormBlock(Block):
    def __init__(self, *, mixer_norm: Norm, mixer: Mixer, ffn_norm: Norm, ffn: FeedForward,
                 act_dtype: torch.dtype = torch.bfloat16):
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn
        self.act_dtype = act_dtype

    def forward(self, ctx: StepContext, slot: LayerSlot, x: torch.Tensor, pending: Optional[torch.Tensor]):
        h, _ = self.mixer_norm.apply(x, pending, rows=None, out_dtype=self.act_dtype)
        mixed = self.mixer.forward(ctx, slot, h)
        h, h32 = self.ffn_norm.apply(x, mixed, rows=None, out_dtype=self.act_dtype,
                                     want_fp32=self.ffn.wants_fp32_input)
        return x, self.ffn.forward(ctx, h, h32)
