"""Dense SwiGLU feed-forward: down( silu(gate(x)) * up(x) ), added into the
residual stream (crates/janus-engine/src/model/block.rs:383-455; SiLU as
x/(1+exp(-x)), crates/janus-engine/src/compute/shaders/activations.wgsl:20-35)."""
from __future__ import annotations

import torch

from .base import FeedForward, register_part
from .linear import GatedLinear, Linear


class SwiGLUFeedForward(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int,
                 dtype: torch.dtype = torch.bfloat16, device: torch.device = torch.device("cuda")):
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.dtype, self.device = dtype, device
        self.gate_up = GatedLinear(hidden_size, intermediate_size, dtype, device)
        self.down = Linear(intermediate_size, hidden_size, dtype, device, name="down")

    def weight_shapes(self):
        return {"gate": ((self.intermediate_size, self.hidden_size), "normal"),
                "up": ((self.intermediate_size, self.hidden_size), "normal"),
                "down": ((self.hidden_size, self.intermediate_size), "normal")}

    def load(self, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> None:
        self.gate_up.load(gate, up)
        self.down.load([down])

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx) -> None:
        act = ctx.workspace.get("ffn_act", (x.shape[0], self.intermediate_size), self.dtype)
        self.gate_up.forward(x, act, ctx)
        self.down.forward_add(act, residual)


register_part("feed_forward", "swiglu", SwiGLUFeedForward)
