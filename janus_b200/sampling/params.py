"""Sampling options with the reference's names and meanings
(`SamplerConfig`, crates/janus-engine/src/model/sampler.rs:20-39, defaults 50-61).

One default differs: `repetition_penalty` is 1.0 (off) here and 1.15 in the
reference, so that temperature 0 is a pure argmax.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplerConfig:
    temperature: float = 0.0          # 0 = greedy argmax (sampler.rs:200-206)
    top_k: int = 0                    # 0 = off; applied to the logits before the temperature (sampler.rs:623-626)
    top_p: float = 1.0                # 1 = off; nucleus over the probabilities (sampler.rs:637-642)
    repetition_penalty: float = 1.0   # over the tokens generated so far (sampler.rs:599-613)
    beam_width: int = 1               # the reference has no beam loop either (sampler.rs:804-847); only 1 is taken
    max_tokens: int = 128             # new tokens per sequence at most (sampler.rs:31-38)

    def validate(self) -> None:
        if self.temperature < 0.0:
            raise ValueError(f"temperature must not be negative, got {self.temperature}")
        if self.top_k < 0:
            raise ValueError(f"top_k must not be negative, got {self.top_k}")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError(f"top_p must lie in (0, 1], got {self.top_p}")
        if not self.repetition_penalty > 0.0:
            raise ValueError(f"repetition_penalty must be positive, got {self.repetition_penalty}")
        if self.beam_width != 1:
            raise ValueError("beam search is not built (beam_width must be 1)")
        if self.max_tokens < 0:
            raise ValueError(f"max_tokens must not be negative, got {self.max_tokens}")
