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

    def reset_row(self, row: int) -> None:
        if self.counts is not None:
            self.counts[row].zero_()

    def sample(self, logits: torch.Tensor, seq_ids: torch.Tensor, steps: torch.Tensor,
               count_rows: Optional[torch.Tensor]) -> torch.Tensor:
        """logits float32 [B, V]; seq_ids, steps, count_rows int32 [B] on the device.
        Returns int32 [B] token ids on the device."""
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=self.device)
        c = self.config
        ops.sample(logits, out, c.temperature, c.top_k, c.top_p, c.repetition_penalty, self.counts,
                   count_rows if self.counts is not None else None, self.seed, seq_ids, steps)
        return out
