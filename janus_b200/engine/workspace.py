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
        self._views: Dict[Tuple[str, torch.dtype, tuple], torch.Tensor] = {}   # asked for on every launch
        self.generation = 0

    def get(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        shape = tuple(shape)
        view = self._views.get((name, dtype, shape))
        if view is not None:
            return view
        n = 1
        for s in shape:
            n *= int(s)
        key = (name, dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < n:
            buf = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self._buffers[key] = buf
            self.generation += 1
            for k in [k for k in self._views if k[0] == name and k[1] == dtype]:
                del self._views[k]           # views of the buffer that was let go
        if len(self._views) > 4096:
            self._views.clear()
        view = self._views[(name, dtype, shape)] = buf[:n].view(*shape)
        return view

    def bytes_held(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())
