"""Sampling on the device: one kernel launch per step for all rows."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .params import SamplerConfig


class DeviceSampler:
    """Holds what sampling needs between steps: for a repetition penalty, a
    table [rows, vocab] counting each row's generated tokens."""

    def __init__(self, config: SamplerConfig, vocab_size: int, max_rows: int, seed: int, device: torch.device):
        config.validate()
        self.config, self.vocab_size, self.seed, self.device = config, vocab_size, int(seed), device
        self.counts: Optional[torch.Tensor] = None
        if config.repetition_penalty != 1.0:
            self.counts = torch.zeros((max_rows, vocab_size), dtype=torch.int32, device=device)

    def graph_key(self):
        """What a captured launch of this sampler depends on."""
        c = self.config
        return (c.temperature, c.top_k, c.top_p, c.repetition_penalty, self.seed,
                0 if self.counts is None else self.counts.data_ptr())

    def reset_row(self, row: int) -> None:
        if self.counts is not None:
            self.counts[row].zero_()

    def sample(self, logits: torch.Tensor, seq_ids: torch.Tensor, steps: torch.Tensor,
               count_rows: Optional[torch.Tensor]) -> torch.Tensor:
        """logits float32 [B, V]; seq_ids, steps, count_rows int32 [B] on the device.
        Returns int32 [B] token ids on the device."""
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=self.device)
        self.sample_into(logits, out, seq_ids, steps, count_rows)
        return out

    def sample_into(self, logits: torch.Tensor, out: torch.Tensor, seq_ids: torch.Tensor, steps: torch.Tensor,
                    count_rows: Optional[torch.Tensor], feedback: Optional[torch.Tensor] = None) -> None:
        """As `sample`, into a given int32 [B] tensor (no allocation: can be captured
        in a CUDA graph).  `feedback` (int32 per cache slot) also receives each
        row's token at its slot `count_rows[b]`, for a next step that reads its
        input tokens on the device."""
        c = self.config
        ops.sample(logits, out, c.temperature, c.top_k, c.top_p, c.repetition_penalty, self.counts,
                   count_rows, self.seed, seq_ids, steps, feedback)
