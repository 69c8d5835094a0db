"""Matrix products y = x W^T with W stored [out, in] (no bias anywhere in the
architecture: crates/janus-engine/src/model/block.rs:239-276 looks none up).

The engine dtype picks the kernel: float32 runs the CUDA-core product (true
32-bit), bfloat16 runs the tcgen05 tensor-core product with float32
accumulation.  Three epilogues: store, add into the float32 residual stream,
and SiLU-gate (for a stacked gate/up weight).
"""
from __future__ import annotations

from typing import Sequence

import torch

from ..kernels import ops


def _to_engine(w: torch.Tensor, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    return w.to(device=device, dtype=dtype).contiguous()


def _check_width(in_features: int, dtype: torch.dtype) -> None:
    """The tensor-core product reads its operands by TMA, whose rows must be multiples of 16 bytes: refuse
    other widths when the model is built, not at the first step."""
    if dtype == torch.bfloat16 and in_features % 8 != 0:
        raise ValueError(f"a bfloat16 product over {in_features} input features is not supported (the width "
                         f"must be a multiple of 8); such a model runs with dtype float32")


class Linear:
    """One weight matrix, possibly the row-wise stack of several tensors of the
    checkpoint (q, k, v stacked so that one product serves all three)."""

    def __init__(self, in_features: int, out_features: int, dtype: torch.dtype, device: torch.device,
                 name: str = ""):
        _check_width(in_features, dtype)
        self.in_features, self.out_features = in_features, out_features
        self.dtype, self.device = dtype, device
        self.name = name     # what a profile of a step calls this product
        self.weight = None   # float32: [out, in] row-major; bfloat16: ops.PackedWeight

    def load(self, tensors: Sequence[torch.Tensor]) -> None:
        parts = [_to_engine(t, self.dtype, self.device) for t in tensors]
        w = parts[0] if len(parts) == 1 else torch.cat(parts, dim=0)
        if tuple(w.shape) != (self.out_features, self.in_features):
            raise ValueError(f"weight of shape {tuple(w.shape)} does not fit "
                             f"({self.out_features}, {self.in_features})")
        # bfloat16 products stream their weights as packed tiles (ops.PackedWeight); float32 stays row-major
        self.weight = ops.pack_weight(w) if self.dtype == torch.bfloat16 else w

    def load_row_major(self, w: torch.Tensor) -> None:
        """A matrix that is already on the device in the engine dtype (a head tied to the embedding: the
        float32 engine uses the embedding's storage as it is, the bfloat16 engine a packed copy)."""
        if tuple(w.shape) != (self.out_features, self.in_features):
            raise ValueError(f"weight of shape {tuple(w.shape)} does not fit ({self.out_features}, {self.in_features})")
        self.weight = ops.pack_weight(w) if self.dtype == torch.bfloat16 else w

    def first_rows(self, rows: int) -> "Linear":
        """The product with the first `rows` output features only (shares storage)."""
        sub = Linear(self.in_features, rows, self.dtype, self.device, self.name)
        sub.weight = self.weight.first_rows(rows) if self.dtype == torch.bfloat16 else self.weight[:rows]
        return sub

    def meets_by_adds(self, tokens: int, y_dtype: torch.dtype) -> bool:
        """Whether `forward` into a float32 `y` for this many tokens cuts K into slices that
        meet in `y` by atomic adds, so that `y` has to be zero beforehand."""
        return (self.dtype != torch.float32 and y_dtype == torch.float32
                and ops.split_k_for(tokens, self.out_features, self.in_features) > 1)

    # y = x W^T, stored in y's dtype (engine dtype, or float32 for logits)
    def forward(self, x: torch.Tensor, y: torch.Tensor, y_is_zero: bool = False) -> None:
        if self.dtype == torch.float32:
            ops.gemm_f32(x, self.weight, y, accumulate=False, label=self.name)
        elif self.meets_by_adds(x.shape[0], y.dtype):
            # few tokens and few output tiles: slices of K run as CTAs of their own and meet in y
            if y_is_zero:
                pass
            elif y.numel() % 4 == 0 and y.data_ptr() % 16 == 0:
                ops.zero_f32(y)
            else:
                y.zero_()
            ops.gemm_bf16(x, self.weight, y, mode="add", label=self.name)
        else:
            ops.gemm_bf16(x, self.weight, y, mode="store", label=self.name)

    # residual += x W^T, the sum made in float32
    def forward_add(self, x: torch.Tensor, residual: torch.Tensor) -> None:
        if self.dtype == torch.float32:
            ops.gemm_f32(x, self.weight, residual, accumulate=True, label=self.name)
        else:
            ops.gemm_bf16(x, self.weight, residual, mode="add", label=self.name)


class GatedLinear:
    """out = silu(x Wg^T) * (x Wu^T) with Wg stacked over Wu
    (crates/janus-engine/src/model/block.rs:383-430)."""

    def __init__(self, in_features: int, out_features: int, dtype: torch.dtype, device: torch.device,
                 name: str = "gate_up"):
        _check_width(in_features, dtype)
        self.in_features, self.out_features = in_features, out_features
        self.dtype, self.device = dtype, device
        self.name = name
        self.weight = None   # float32: [2 * out, in] row-major; bfloat16: a packed gated pair
        self._stacked = None  # bfloat16: the same tiles as one plain matrix (gate rows, then up rows)

    def load(self, gate: torch.Tensor, up: torch.Tensor) -> None:
        g, u = _to_engine(gate, self.dtype, self.device), _to_engine(up, self.dtype, self.device)
        for t in (g, u):
            if tuple(t.shape) != (self.out_features, self.in_features):
                raise ValueError(f"gate/up weight of shape {tuple(t.shape)} does not fit "
                                 f"({self.out_features}, {self.in_features})")
        self.weight = ops.pack_gated(g, u) if self.dtype == torch.bfloat16 else torch.cat([g, u], dim=0)
        self._stacked = None

    def forward(self, x: torch.Tensor, out: torch.Tensor, ctx) -> None:
        if self.dtype == torch.float32:
            gu = ctx.workspace.get("gate_up", (x.shape[0], 2 * self.out_features), torch.float32)
            ops.gemm_f32(x, self.weight, gu, accumulate=False, label=self.name)
            ops.swiglu(gu, out)
        elif ops.gated_runs_unfused(x.shape[0], self.out_features):
            # few tokens, narrow layer: twice the tiles stream the weights as a plain product; the gate is applied after
            if self._stacked is None:
                self._stacked = self.weight.stacked()
            gu = ctx.workspace.get("gate_up", (x.shape[0], self._stacked.rows), torch.float32)
            ops.gemm_bf16(x, self._stacked, gu, mode="store", pair=False, label=self.name)
            ops.swiglu_f32_to_bf16(gu, out, 128 * self.weight.up_tile_offset)
        else:
            ops.gemm_bf16(x, self.weight, out, mode="swiglu", label=self.name)
