"""Grouped-query attention over the paged cache.

q, k, v projections as one stacked product; rotary positions on q and k fused
with the append of k (rotated) and v to the cache; causal attention of every
new token over its sequence's cached keys (optionally only the last `window`);
output projection added into the residual stream.  Formulas:
crates/janus-engine/src/model/block.rs:239-363 and
crates/janus-engine/src/compute/shaders/attention.wgsl:96-115,170-185
(kv head of query head h is floor(h*nkv/nh); score = dot * 1/sqrt(head_dim)).
"""
from __future__ import annotations

import math
import os
from typing import Optional

import torch

from ..kernels import ops
from .base import KVSpec, Mixer, PartSpec, register_part, shared_part
from .linear import Linear


# JANUS_FUSED_DECODE=0 keeps rotation and cache append in a kernel of their own for decode steps too
_FUSED_DECODE = os.environ.get("JANUS_FUSED_DECODE", "1") != "0"


def _check_kernel_limits(num_heads: int, num_kv_heads: int, head_dim: int, dtype: torch.dtype) -> None:
    """Refuse, when the part is built, the sizes that the attention kernels refuse at a step."""
    if head_dim < 1 or head_dim > ops.ATTENTION_MAX_HEAD_DIM:
        raise ValueError(f"head_dim {head_dim} is not supported: the attention kernels take head sizes up to "
                         f"{ops.ATTENTION_MAX_HEAD_DIM}")
    if dtype == torch.bfloat16:
        if head_dim % 8:
            raise ValueError(f"head_dim {head_dim} is not supported in bfloat16 (it must be a multiple of 8: "
                             f"cache rows are read in 16-byte pieces); such a model runs with dtype float32")
        group = num_heads // num_kv_heads
        if (group > ops.ATTENTION_BF16_MAX_GROUP
                and not ops.attention_tc_supported(num_heads, num_kv_heads, head_dim)):
            raise ValueError(f"{group} query heads per key/value head are not supported in bfloat16 with head_dim "
                             f"{head_dim} (at most {ops.ATTENTION_BF16_MAX_GROUP}); such a model runs with dtype float32")


class GQAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position: Optional[PartSpec] = None, window: int = 0,
                 dtype: torch.dtype = torch.bfloat16, device: torch.device = torch.device("cuda")):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {num_kv_heads} key/value heads")
        self.hidden_size, self.nh, self.nkv, self.hd = hidden_size, num_heads, num_kv_heads, head_dim
        self.window = int(window)
        self.dtype, self.device = dtype, device
        self.scale = 1.0 / math.sqrt(head_dim)          # crates/janus-engine/src/compute/ops/attention.rs:98
        _check_kernel_limits(num_heads, num_kv_heads, head_dim, dtype)
        # layers that name the same position encoding share one object (one table on the device)
        self.position = shared_part("position", position, dtype, device) if position is not None else None
        self.q_width, self.kv_width = num_heads * head_dim, num_kv_heads * head_dim
        self.qkv = Linear(hidden_size, self.q_width + 2 * self.kv_width, dtype, device, name="qkv")
        self.q_only: Optional[Linear] = None             # view of the q rows, for layers that read another cache
        self.o = Linear(self.q_width, hidden_size, dtype, device, name="o")

    def cache_spec(self) -> KVSpec:
        return KVSpec(self.nkv, self.hd, self.window)

    def limit_positions(self, n: int) -> None:
        limit = getattr(self.position, "limit_positions", None)
        if limit is not None:
            limit(n)

    def weight_shapes(self):
        return {"q": ((self.q_width, self.hidden_size), "normal"),
                "k": ((self.kv_width, self.hidden_size), "normal"),
                "v": ((self.kv_width, self.hidden_size), "normal"),
                "o": ((self.hidden_size, self.q_width), "normal")}

    def load(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o: torch.Tensor) -> None:
        self.qkv.load([q, k, v])
        self.o.load([o])
        self.q_only = self.qkv.first_rows(self.q_width)

    def scratch_to_clear(self, ctx, tokens: int, writes_cache: bool = True) -> Optional[torch.Tensor]:
        """The q/k/v buffer, if this step's projection adds K slices into it (decode-sized
        steps): the norm before this mixer clears it in the same launch."""
        proj = self.qkv if writes_cache else self.q_only
        if proj is None or not proj.meets_by_adds(tokens, torch.float32):
            return None
        if self._projection_writes_cache(ctx, tokens, writes_cache):
            return None
        qkv = ctx.workspace.get("qkv", (tokens, proj.out_features), torch.float32)
        return qkv if qkv.numel() % 4 == 0 else None

    def _projection_writes_cache(self, ctx, tokens: int, writes_cache: bool) -> bool:
        """Whether this step's q/k/v projection rotates and appends to the cache in its own epilogue
        (prompts of bfloat16 models whose positions are a rotation by table)."""
        table = self.position.fused_rotary_table() if self.position is not None else None
        return (self.dtype == torch.bfloat16 and writes_cache and table is not None and not ctx.is_decode
                and ops.gemm_qkv_rope_supported(tokens, self.hd))

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, cache_view, writes_cache: bool = True,
                scratch_cleared: bool = False) -> None:
        T = x.shape[0]
        ws = ctx.workspace
        group = cache_view.group
        table = self.position.fused_rotary_table() if self.position is not None else None
        if self._projection_writes_cache(ctx, T, writes_cache):
            # a prompt: the projection's epilogue rotates q and k and appends k and v to the cache
            q = ws.get("q_rot", (T, self.q_width), self.dtype)
            ops.gemm_qkv_rope_cache(x, self.qkv.weight, q, table, ctx.positions, group.dest_rows, cache_view.k,
                                    cache_view.v, self.nh, self.nkv, self.hd, group.page_size)
            self._attend_prompt(q, residual, ctx, cache_view)
            return
        proj = self.qkv if writes_cache else self.q_only
        # the projection's float32 accumulators go straight into the rotation
        qkv = ws.get("qkv", (T, proj.out_features), torch.float32)
        proj.forward(x, qkv, y_is_zero=scratch_cleared)
        custom_positions = self.position is not None and table is None
        if custom_positions:
            self.position.apply(qkv[:, : self.q_width], self.nh, self.hd, ctx.positions)
            if writes_cache:
                self.position.apply(qkv[:, self.q_width: self.q_width + self.kv_width], self.nkv, self.hd,
                                    ctx.positions)
        attn = ws.get("attn_out", (T, self.q_width), self.dtype)
        if ctx.is_decode and self.dtype == torch.bfloat16 and _FUSED_DECODE and not custom_positions:
            # one token per sequence: rotation and cache append happen inside the attention kernel
            # (one launch and one round trip of q less)
            ops.attention_bf16_decode(None, cache_view.k, cache_view.v, attn, group.block_table, ctx.kv_len,
                                      self.nh, self.nkv, self.hd, group.page_size, self.window, self.scale,
                                      ctx.workspace, ctx.max_kv_len_bound, qkv=qkv, cos_sin=table,
                                      dest=group.dest_rows if writes_cache else None, write_kv=writes_cache)
            self.o.forward_add(attn, residual)
            return
        q = ws.get("q_rot", (T, self.q_width), self.dtype)
        ops.rope_cache_write(qkv, q, table, ctx.positions, group.dest_rows if writes_cache else None,
                             cache_view.k if writes_cache else None, cache_view.v if writes_cache else None,
                             self.nh, self.nkv, self.hd, group.page_size, write_kv=writes_cache)
        if self.dtype == torch.float32:
            ops.attention_f32(q, cache_view.k, cache_view.v, attn, group.block_table, ctx.token_seq,
                              ctx.positions, self.nh, self.nkv, self.hd, group.page_size, self.window,
                              self.scale)
        elif ctx.is_decode:
            ops.attention_bf16_decode(q, cache_view.k, cache_view.v, attn, group.block_table, ctx.kv_len,
                                      self.nh, self.nkv, self.hd, group.page_size, self.window, self.scale,
                                      ctx.workspace, ctx.max_kv_len_bound)
        else:
            self._attend_prompt(q, residual, ctx, cache_view)
            return
        self.o.forward_add(attn, residual)

    def _attend_prompt(self, q: torch.Tensor, residual: torch.Tensor, ctx, cache_view) -> None:
        """bfloat16 attention of several new tokens per sequence over the cache, then the output projection."""
        group = cache_view.group
        attn = ctx.workspace.get("attn_out", (q.shape[0], self.q_width), self.dtype)
        if ops.attention_tc_supported(self.nh, self.nkv, self.hd):
            # head sizes up to 128: flash attention on the tcgen05 tensor cores
            ops.attention_tc_prefill(q, cache_view.k, cache_view.v, attn, group.block_table, ctx.q_start,
                                     ctx.kv_len, ctx.n_seqs, ctx.max_q_len, self.nh, self.nkv, self.hd,
                                     group.page_size, self.window, self.scale)
        else:
            ops.attention_bf16_prefill(q, cache_view.k, cache_view.v, attn, group.block_table, ctx.q_start,
                                       ctx.kv_len, ctx.n_seqs, ctx.max_q_len, self.nh, self.nkv, self.hd,
                                       group.page_size, self.window, self.scale)
        self.o.forward_add(attn, residual)


register_part("mixer", "gqa_attention", GQAttention)
