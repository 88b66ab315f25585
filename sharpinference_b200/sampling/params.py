"""``SamplingParams``: how the next token is chosen, with the reference's names and meanings
(src/SharpInference.Engine/Sampler.cs:648-893).

* ``temperature``: 0 or below means greedy; otherwise logits are divided by it (default 1.0; the
  command line's ``--temp`` defaults to 0.7 like the reference's).
* ``top_k`` (0 = off), ``top_p`` (1.0 = off), ``min_p`` (0 = off): filters applied in that order
  after the softmax, as in the reference's full-vocabulary path (:71-107).
* ``repetition_penalty`` (1.0 = off: a seen token's logit is divided by it if positive, multiplied
  if negative, once per distinct token), ``frequency_penalty`` and ``presence_penalty`` (subtracted:
  ``count * frequency + presence``), over the last ``penalty_last_n`` tokens (0 = all), the window
  seeded from the prompt's tail when ``penalty_seed_from_prompt`` (:405-432).
* ``logit_bias``: token id -> additive bias before the temperature.
* ``max_new_tokens`` (512); ``stop_token_ids`` replaces the model's end-of-generation set,
  ``additional_stop_token_ids`` is united with it (:884-892).
* ``seed``: the request's random stream; ``None`` draws a fresh one.  The reference seeds only
  from the command line (src/SharpInference.Cli/RunCommand.cs:1234).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Sequence, Tuple


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    penalty_last_n: int = 256
    penalty_seed_from_prompt: bool = True
    logit_bias: Optional[Dict[int, float]] = None
    max_new_tokens: int = 512
    stop_token_ids: Optional[Sequence[int]] = None
    additional_stop_token_ids: Optional[Sequence[int]] = None
    seed: Optional[int] = None

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    @property
    def has_penalties(self) -> bool:
        return self.repetition_penalty != 1.0 or self.frequency_penalty != 0.0 or self.presence_penalty != 0.0

    def resolve_stop_set(self, end_of_generation: Sequence[int]) -> Tuple[int, ...]:
        """``stop_token_ids`` replaces the model's set; ``additional_stop_token_ids`` is added to
        whichever of the two applies."""
        base = tuple(self.stop_token_ids) if self.stop_token_ids is not None else tuple(end_of_generation)
        if self.additional_stop_token_ids:
            return tuple(sorted(set(base) | set(self.additional_stop_token_ids)))
        return base
