"""Arrangement of a layer's parts.  Pre-norm, as the reference's block:
h1 = x + mixer(norm1(x)); out = h1 + feed_forward(norm2(h1))
(crates/janus-engine/src/model/block.rs:223-233,355-380,447-455).  The parts
add into the float32 residual stream themselves."""
from __future__ import annotations

import torch

from .base import register_part


class PreNormBlock:
    """`parts`: mixer_norm and mixer, and, unless the layer has no feed-forward,
    feed_forward_norm and feed_forward."""

    def __init__(self, parts: dict, hidden_size: int, dtype: torch.dtype):
        unknown = set(parts) - {"mixer_norm", "mixer", "feed_forward_norm", "feed_forward"}
        if unknown:
            raise ValueError(f"the pre_norm arrangement has no use for the parts {sorted(unknown)}")
        try:
            self.mixer_norm, self.mixer = parts["mixer_norm"], parts["mixer"]
            self.feed_forward = parts.get("feed_forward")
            self.feed_forward_norm = parts["feed_forward_norm"] if self.feed_forward is not None else None
        except KeyError as e:
            raise ValueError(f"the pre_norm arrangement needs the part {e.args[0]!r}") from None
        self.hidden_size, self.dtype = hidden_size, dtype

    def forward(self, residual: torch.Tensor, ctx, cache_view, writes_cache: bool = True) -> None:
        x = ctx.workspace.get("normed", (residual.shape[0], self.hidden_size), self.dtype)
        # a mixer may name a scratch buffer that it wants zeroed; the norm before it does that in passing
        wants = getattr(self.mixer, "scratch_to_clear", None)
        scratch = wants(ctx, residual.shape[0], writes_cache) if wants is not None else None
        if scratch is not None:
            self.mixer_norm.forward(residual, x, clear=scratch)
            self.mixer.forward(x, residual, ctx, cache_view, writes_cache, scratch_cleared=True)
        else:
            self.mixer_norm.forward(residual, x)
            self.mixer.forward(x, residual, ctx, cache_view, writes_cache)
        if self.feed_forward is None:
            return
        self.feed_forward_norm.forward(residual, x)
        self.feed_forward.forward(x, residual, ctx)


register_part("arrangement", "pre_norm", PreNormBlock)
