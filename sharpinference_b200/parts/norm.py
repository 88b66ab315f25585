"""Norm parts: RMSNorm with a weight, and the weightless L2 norm used on q and k per head.

RMSNorm: ``x * rsqrt(mean(x^2) + eps) * w`` (src/SharpInference.Cpu/SimdKernels.cs:4209-4246);
the weightless form drops ``w`` (src/SharpInference.Cpu/SimdKernels.cs:4252-4283).  The sum of
squares, the rsqrt and the scaling are float32.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Norm, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    def __init__(self, weight: torch.Tensor, eps: float):
        self.weight = weight
        self.eps = float(eps)

    def apply(self, x, delta, *, rows=None, out_dtype=torch.bfloat16, want_fp32=False):
        return ops.add_rmsnorm(x, delta, self.weight, self.eps, out_dtype, rows=rows, want_fp32=want_fp32)


@register_part("norm", "l2")
class L2Norm(Norm):
    """``x * rsqrt(mean(x^2) + eps)`` over the last axis, no weight.  As the q/k norm after a rotary encoding
    the attention mixer runs it fused with the rotation and the cache write (``fuses_into_rotation``); anywhere
    else it is a launch of its own like every norm."""

    fuses_into_rotation = True

    def __init__(self, eps: float):
        self.eps = float(eps)

    def apply(self, x, delta, *, rows=None, out_dtype=torch.bfloat16, want_fp32=False):
        return ops.add_rmsnorm(x, delta, None, self.eps, out_dtype, rows=rows, want_fp32=want_fp32)
