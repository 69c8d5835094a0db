"""Scratch tensors of a step, kept between steps.  A buffer grows when a step
needs more; growth moves it, which `generation` records so that captured CUDA
graphs (which hold addresses) are thrown away."""
from __future__ import annotations

from typing import Dict, Tuple

import torch


class Workspace:
    def __init__(self, device: torch.device):
        self.device = device
        self._buffers: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        self.generation = 0

    def get(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        key = (name, dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < n:
            buf = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self._buffers[key] = buf
            self.generation += 1
        return buf[:n].view(*shape)

    def bytes_held(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())
