"""The sampler: one next token for every row of logits, on the device.

Greedy rows (temperature <= 0) take the arg-max of the raw logits, the lowest index among ties, before
any bias or penalty, as the reference does (src/SharpInference.Engine/Sampler.cs:17-18); other rows go
through logit bias, window penalties, temperature, softmax, top-k, min-p, top-p and an inverse-CDF draw
(``csrc/sampling.cu``, following src/SharpInference.Engine/Sampler.cs:15-107).  Each request owns
a counter-based random stream: draw ``n`` of a request with seed ``s`` is
``uniform(splitmix64(s, n))``, so its tokens do not depend on what else is in the batch.
"""
from __future__ import annotations

import random
from collections import Counter
from dataclasses import dataclass, field
from typing import List, Sequence

import torch

from ..kernels import ops
from .params import SamplingParams

_MASK64 = (1 << 64) - 1


def splitmix64(seed: int, counter: int) -> int:
    z = (seed * 0x9E3779B97F4A7C15 + (counter + 1) * 0xBF58476D1CE4E5B9) & _MASK64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
    return z ^ (z >> 31)


def uniform01(seed: int, counter: int) -> float:
    """A number in (0, 1) with 24 random bits, exact in float32."""
    return ((splitmix64(seed, counter) >> 40) + 0.5) / float(1 << 24)


@dataclass
class SamplerState:
    """Per-request sampling state: parameters, random stream, penalty window."""

    params: SamplingParams
    seed: int = 0
    draws: int = 0
    window: List[int] = field(default_factory=list)

    @classmethod
    def start(cls, params: SamplingParams, prompt: Sequence[int]) -> "SamplerState":
        seed = params.seed if params.seed is not None and params.seed >= 0 else random.getrandbits(63)
        st = cls(params=params, seed=int(seed))
        if params.has_penalties and params.penalty_seed_from_prompt:
            st.window = list(prompt[-params.penalty_last_n:] if params.penalty_last_n > 0 else prompt)
        return st

    def observe(self, token: int) -> None:
        if self.params.has_penalties:
            self.window.append(token)
            n = self.params.penalty_last_n
            if n > 0 and len(self.window) > n:
                del self.window[: len(self.window) - n]


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, states: Sequence[SamplerState]) -> List[int]:
        """``logits`` float32 [R, V] on the device (edited in place by bias and penalties);
        one state per row.  Returns R token ids and advances each state's stream and window."""
        R = logits.shape[0]
        if R != len(states):
            raise ValueError(f"{R} rows of logits for {len(states)} requests")
        dev = self.device
        bias_rows, bias_tok, bias_val = [], [], []
        pen_rows, pen_tok, pen_cnt = [], [], []
        for r, st in enumerate(states):
            p = st.params
            if p.greedy:                    # the arg-max of the raw logits: no bias, no penalty
                continue
            if p.logit_bias:
                for tok, b in p.logit_bias.items():
                    bias_rows.append(r); bias_tok.append(int(tok)); bias_val.append(float(b))
            if p.has_penalties and st.window:
                for tok, cnt in Counter(st.window).items():
                    pen_rows.append(r); pen_tok.append(int(tok)); pen_cnt.append(int(cnt))
        if bias_rows:
            ops.add_logit_bias(logits, torch.tensor(bias_rows, dtype=torch.int32, device=dev),
                               torch.tensor(bias_tok, dtype=torch.int32, device=dev),
                               torch.tensor(bias_val, dtype=torch.float32, device=dev))
        if pen_rows:
            f = lambda name: torch.tensor([getattr(s.params, name) for s in states], dtype=torch.float32, device=dev)
            ops.apply_penalties(logits, torch.tensor(pen_rows, dtype=torch.int32, device=dev),
                                torch.tensor(pen_tok, dtype=torch.int32, device=dev),
                                torch.tensor(pen_cnt, dtype=torch.int32, device=dev),
                                f("repetition_penalty"), f("frequency_penalty"), f("presence_penalty"))
        if all(st.params.greedy for st in states):
            picked = ops.argmax_rows(logits)
        else:
            host = torch.tensor(
                [[st.params.temperature, st.params.top_p, st.params.min_p,
                  0.0 if st.params.greedy else uniform01(st.seed, st.draws)] for st in states],
                dtype=torch.float32).t().contiguous().to(dev)
            top_k = torch.tensor([st.params.top_k for st in states], dtype=torch.int32, device=dev)
            picked = ops.sample_rows(logits, host[0], top_k, host[1], host[2], host[3],
                                     any_top_k=any(0 < st.params.top_k for st in states),
                                     any_top_p=any(0.0 < st.params.top_p < 1.0 for st in states))
        tokens = picked.tolist()
        for st, tok in zip(states, tokens):
            if not st.params.greedy:
                st.draws += 1
            st.observe(tok)
        return tokens
