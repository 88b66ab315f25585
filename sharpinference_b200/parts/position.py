"""Position encodings.

``RotaryEncoding`` rotates pairs of a head's elements by ``position * inv_freq[j]``.  Llama 4
pairs neighbours, ``(2j, 2j+1)`` (src/SharpInference.Cpu/SimdKernels.cs:4591-4629; the
architecture is absent from the reference's list of half-split models,
src/SharpInference.Core/ModelGraph.cs:308-328).  The frequencies are
``theta^(-2j/d)`` (src/SharpInference.Cpu/SimdKernels.cs:4789-4811), optionally rescaled by the
"llama3" rule, which the reference only knows as a stored table of divisors
(src/SharpInference.Engine/ForwardPass.cs:259-276):

    wavelength = 2 pi / f
    wavelength < L / high_freq_factor  ->  f                      (short waves stay)
    wavelength > L / low_freq_factor   ->  f / factor             (long waves are stretched)
    otherwise                           ->  (1 - s) f / factor + s f,
                                            s = (L / wavelength - low) / (high - low)

with ``L = original_max_position_embeddings``.  The table is float32 and built once; the angle
``position * inv_freq`` and its sine and cosine are float32 in the kernel.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from .base import PositionEncoding, register_part


def rotary_inv_freq(head_dim: int, theta: float, scaling=None) -> torch.Tensor:
    """float32 ``[head_dim / 2]`` rotation frequencies (CPU tensor).

    The unscaled frequency is the reference's ``1 / pow(theta, 2 j / d)`` in float32
    (src/SharpInference.Cpu/SimdKernels.cs:4795); the rescaling follows the three cases of the
    module docstring, one frequency at a time.
    """
    pairs = head_dim // 2
    two_j_over_d = torch.arange(pairs, dtype=torch.float32) * 2.0 / float(head_dim)
    freqs = 1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float32), two_j_over_d)
    if scaling is None:
        return freqs
    span = float(scaling.original_max_position_embeddings)
    low, high, factor = float(scaling.low_freq_factor), float(scaling.high_freq_factor), float(scaling.factor)
    out = torch.empty_like(freqs)
    for j in range(pairs):
        f = freqs[j]                                   # float32 scalar tensor: the arithmetic stays float32
        turns = span * f / (2.0 * math.pi)             # L / wavelength
        if turns > high:                               # wavelength < L / high: short waves stay
            out[j] = f
        elif turns < low:                              # wavelength > L / low: long waves are stretched
            out[j] = f / factor
        elif high == low:                              # the band between them is empty
            out[j] = f
        else:
            s = (turns - low) / (high - low)
            out[j] = (1.0 - s) * f / factor + s * f
    return out


@register_part("position", "rotary")
class RotaryEncoding(PositionEncoding):
    def __init__(self, inv_freq: torch.Tensor, pairing: str = "interleaved"):
        if pairing not in ("interleaved", "halves"):
            raise ValueError(f"rotary pairing '{pairing}' is not one of interleaved, halves")
        self.inv_freq = inv_freq
        self.pairing = pairing

    def rotary(self) -> Optional[Tuple[torch.Tensor, str]]:
        return self.inv_freq, self.pairing


@register_part("position", "none")
class NoPositionEncoding(PositionEncoding):
    """Layers that see positions only through the causal mask."""

    def rotary(self):
        return None

    def apply(self, ctx, q, k):
        return None
