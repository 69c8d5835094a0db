"""Rotary positions: half-split pairs (i, i + head_dim/2) rotated by the angle
position * inv_freq_i, inv_freq_i = 1 / theta^(2i/head_dim), all in float32;
cos and sin are tabulated on the host once, as the reference does
(crates/janus-engine/src/model/transformer/constructor.rs:454-489; pairing in
crates/janus-engine/src/compute/shaders/rope.wgsl:55-76).  The reference
hard-codes theta = 10000 and has no frequency scaling
(crates/janus-engine/src/model/config.rs:299); here both are parameters, with
the "llama3" rule of config.json's `rope_scaling`.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .base import PositionEncoding, register_part


def llama3_scaled(inv_freq: torch.Tensor, factor: float, low_freq_factor: float, high_freq_factor: float,
                  original_max_position_embeddings: int) -> torch.Tensor:
    """Frequencies with wavelength above original/low are divided by `factor`,
    those below original/high are kept, the band between is blended linearly
    in original/wavelength."""
    f = inv_freq.to(torch.float32)
    wavelen = (2.0 * math.pi) / f
    low_wavelen = original_max_position_embeddings / low_freq_factor
    high_wavelen = original_max_position_embeddings / high_freq_factor
    smooth = (original_max_position_embeddings / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor)
    blended = (1.0 - smooth) * f / factor + smooth * f
    out = torch.where(wavelen < high_wavelen, f, torch.where(wavelen > low_wavelen, f / factor, blended))
    return out.to(torch.float32)


class RotaryEncoding(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, max_positions: int, scaling: Optional[dict] = None,
                 dtype: torch.dtype = torch.float32, device: torch.device = torch.device("cpu")):
        if head_dim % 2:
            raise ValueError(f"rotary positions need an even head_dim, got {head_dim}")
        self.head_dim, self.theta, self.max_positions = int(head_dim), float(theta), int(max_positions)
        self.scaling = scaling
        self.device = device
        exponent = torch.arange(0, head_dim, 2, dtype=torch.float32) / float(head_dim)
        inv_freq = 1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float32), exponent)
        if scaling is not None:
            inv_freq = llama3_scaled(inv_freq, **{k: v for k, v in scaling.items() if k != "rope_type"})
        self.inv_freq = inv_freq
        self._limit = self.max_positions
        self._table: Optional[torch.Tensor] = None

    def limit_positions(self, n: int) -> None:
        """Positions beyond `n` are never asked for (the engine's longest sequence):
        the table gets no more rows than that.  Several engines may share this
        object; the largest limit counts, and a table that is too short is made
        anew (the engine that asked for less has captured no step yet)."""
        n = min(int(n), self.max_positions)
        if self._table is None:
            self._limit = n
        elif n > self._table.shape[0]:
            self._limit, self._table = n, None

    @property
    def table(self) -> torch.Tensor:
        """cos and sin of position * inv_freq, float32 [positions, head_dim/2, 2],
        tabulated on the host at first use and shared by every layer."""
        if self._table is None:
            angle = torch.arange(self._limit, dtype=torch.float32)[:, None] * self.inv_freq[None, :]
            self._table = torch.stack([torch.cos(angle), torch.sin(angle)], dim=-1).contiguous().to(self.device)
        return self._table

    def fused_rotary_table(self) -> torch.Tensor:
        return self.table


class NoPositions(PositionEncoding):
    """A mixer whose order information comes from elsewhere."""

    def __init__(self, dtype=None, device=None, **_):
        pass

    def apply(self, x, heads, head_dim, positions) -> None:
        return None


register_part("position", "rotary", RotaryEncoding)
register_part("position", "none", NoPositions)
