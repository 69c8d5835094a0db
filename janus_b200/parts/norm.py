"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * gamma, statistics in float32
(crates/janus-engine/src/compute/shaders/activations.wgsl:81-133).  The weight
keeps the dtype it was stored in (the reference keeps 1-D tensors in f32,
crates/janus-engine/src/compute/engine.rs:448-470)."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import Norm, register_part


class RMSNorm(Norm):
    def __init__(self, width: int, eps: float, dtype: torch.dtype, device: torch.device):
        self.width, self.eps = int(width), float(eps)
        self.dtype, self.device = dtype, device
        self.gamma: Optional[torch.Tensor] = None

    def weight_shapes(self):
        return {"gamma": ((self.width,), "ones")}

    def load(self, gamma: torch.Tensor) -> None:
        if tuple(gamma.shape) != (self.width,):
            raise ValueError(f"norm weight of shape {tuple(gamma.shape)} does not fit ({self.width},)")
        if self.dtype == torch.float32:
            gamma = gamma.to(torch.float32)
        self.gamma = gamma.to(self.device).contiguous()

    def forward(self, x: torch.Tensor, out: torch.Tensor, row_index: Optional[torch.Tensor] = None,
                clear: Optional[torch.Tensor] = None) -> None:
        """`clear`: a float32 scratch tensor of the part that runs next, set to zero by the same launch."""
        ops.rmsnorm(x, self.gamma, self.eps, out, row_index, clear)


register_part("norm", "rms_norm", RMSNorm)
