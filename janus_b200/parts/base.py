"""Interfaces of the parts a decoder is put together from, their registries,
and the data that describes a model (`ModelSpec`).

A model is data: for each layer a mixer, a feed-forward, norms and their
arrangement, each named by a registered kind with its sizes and constants as
parameters and the checkpoint names of its weights; plus the order in which
layers run.  No part knows which model it is in.

Interfaces
----------
Norm          load(gamma); forward(x_f32[rows,H] , out[rows,H], row_index=None)
Position      fused_rotary_table() -> [positions, head_dim/2, 2] float32 or None;
              apply(x[T, heads*head_dim], heads, head_dim, positions) in place (only if no table)
Mixer         cache_spec() -> KVSpec | StateSpec | None
              forward(x[T,H], residual_f32[T,H], ctx, cache_view, writes_cache): adds its output into residual
FeedForward   forward(x[T,H], residual_f32[T,H], ctx): adds its output into residual
Transform     forward(t, ctx): changes a whole tensor of the model in place: the residual stream after the
              embedding (scale it, add positions) or the logits (scale, soft-cap); see `ModelSpec`
Arrangement   factory(parts: {role: part}, hidden_size, dtype);
              forward(residual_f32[T,H], ctx, cache_view, writes_cache)
all parts     weight_shapes() -> {parameter: (shape, init)};  load(**tensors)

A part's `forward` only enqueues device work on the current stream and keeps no
host-side record of what it has seen: a decode step may be recorded into a CUDA
graph (the recording call runs no device work) and replayed many times.

The residual stream is float32 in both engine dtypes, so the residual sum is
always made in 32 bits; `x` is the normed layer input in the engine dtype.
"""
from __future__ import annotations

import weakref
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple, Union

import torch


# --------------------------------------------------------------------------
# what a mixer needs from the cache
# --------------------------------------------------------------------------
@dataclass(frozen=True)
class KVSpec:
    """Keys and values per token.  window = 0 keeps every key; window = w keeps
    the last w keys (the query's own position included)."""
    n_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateSpec:
    """Per-sequence state of fixed size, float32, zeroed when a slot is taken."""
    shape: Tuple[int, ...]


CacheSpec = Union[KVSpec, StateSpec, None]


# --------------------------------------------------------------------------
# model description
# --------------------------------------------------------------------------
@dataclass(frozen=True)
class PartSpec:
    kind: str                                   # a registered kind
    params: Dict[str, Any] = field(default_factory=dict)
    weights: Dict[str, str] = field(default_factory=dict)   # part parameter -> checkpoint tensor name


_ROLE_FAMILIES = (("mixer_norm", "norm"), ("mixer", "mixer"), ("feed_forward_norm", "norm"),
                  ("feed_forward", "feed_forward"))


@dataclass(frozen=True)
class LayerSpec:
    """The parts of one layer by role.  Only the mixer is required; which of the
    others a layer needs is its arrangement's business (a layer without a
    feed-forward leaves it and its norm out).  `extra` names further parts that
    an arrangement of one's own uses, as (role, family, spec): norms after the
    mixer or after the feed-forward, a second feed-forward, ..."""
    mixer: PartSpec
    feed_forward: Optional[PartSpec] = None
    mixer_norm: Optional[PartSpec] = None
    feed_forward_norm: Optional[PartSpec] = None
    arrangement: str = "pre_norm"
    extra: Tuple[Tuple[str, str, PartSpec], ...] = ()

    def parts(self) -> List[Tuple[str, str, PartSpec]]:
        """(role, family, spec) of every part the layer has."""
        out = [(role, family, getattr(self, role)) for role, family in _ROLE_FAMILIES
               if getattr(self, role) is not None]
        roles = {r for r, _, _ in out}
        for role, family, spec in self.extra:
            if role in roles:
                raise ValueError(f"a layer names the role '{role}' twice")
            roles.add(role)
            out.append((role, family, spec))
        return out


@dataclass(frozen=True)
class ScheduleEntry:
    """One place in the order of execution: which layer runs, and whose cache it
    reads (None = its own, written at this place; an earlier place's index = it
    reads that place's keys and values and writes none)."""
    layer: int
    reads_cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    embedding_weight: str
    head_weight: Optional[str]                  # None = tied to the embedding
    max_positions: int
    ignorable_weights: Tuple[str, ...] = ()
    # transforms ("transform" family) of the residual stream after the embedding and of the logits
    # after the head, in order; none in the Llama decoder
    embedding_transforms: Tuple[PartSpec, ...] = ()
    logit_transforms: Tuple[PartSpec, ...] = ()


# --------------------------------------------------------------------------
# registries
# --------------------------------------------------------------------------
_REGISTRIES: Dict[str, Dict[str, Callable[..., Any]]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "arrangement": {}, "transform": {},
}


def register_part(family: str, kind: str, factory: Callable[..., Any]) -> None:
    """`factory(**params, dtype=..., device=...)` builds the part.  `family` is
    one of mixer, feed_forward, norm, position, transform; an arrangement's
    factory takes `(parts, hidden_size, dtype)`."""
    if family not in _REGISTRIES:
        raise KeyError(f"unknown family '{family}' (have {sorted(_REGISTRIES)})")
    _REGISTRIES[family][kind] = factory


def make_part(family: str, spec: PartSpec, dtype: torch.dtype, device: torch.device):
    try:
        factory = _REGISTRIES[family][spec.kind]
    except KeyError:
        raise KeyError(f"no {family} of kind '{spec.kind}' is registered "
                       f"(have {sorted(_REGISTRIES[family])})") from None
    return factory(**spec.params, dtype=dtype, device=device)


_shared: "weakref.WeakValueDictionary[tuple, Any]" = weakref.WeakValueDictionary()


def shared_part(family: str, spec: PartSpec, dtype: torch.dtype, device: torch.device):
    """One object per distinct (family, kind, parameters, dtype, device), for parts
    that never change once built (a position encoding's table): every layer that
    names the same spec gets the same object for as long as one of them lives."""
    key = (family, spec.kind, repr(sorted(spec.params.items())), str(dtype), str(torch.device(device)))
    part = _shared.get(key)
    if part is None:
        part = make_part(family, spec, dtype, device)
        _shared[key] = part
    return part


def registered_parts(family: str) -> List[str]:
    return sorted(_REGISTRIES[family])


# --------------------------------------------------------------------------
# base classes (documentation of the interfaces; parts need not inherit)
# --------------------------------------------------------------------------
class Part:
    def weight_shapes(self) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        """{parameter: (shape, init)} with init "normal" or "ones"."""
        return {}

    def load(self, **tensors: torch.Tensor) -> None:
        if tensors:
            raise TypeError(f"{type(self).__name__} takes no weights, got {sorted(tensors)}")


class Norm(Part):
    def forward(self, x: torch.Tensor, out: torch.Tensor, row_index: Optional[torch.Tensor] = None,
                clear: Optional[torch.Tensor] = None) -> None:
        """out[r] = norm(x[row_index[r]] or x[r]) for the rows of `out` (x float32, out the engine dtype).
        `clear`: a float32 scratch tensor of the part that runs next, to be set to zero on the way (an
        arrangement passes it when that part asks for it)."""
        raise NotImplementedError


class PositionEncoding(Part):
    def fused_rotary_table(self) -> Optional[torch.Tensor]:
        return None

    def apply(self, x: torch.Tensor, heads: int, head_dim: int, positions: torch.Tensor) -> None:
        raise NotImplementedError


class Mixer(Part):
    def cache_spec(self) -> CacheSpec:
        return None

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, cache_view, writes_cache: bool = True) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx) -> None:
        raise NotImplementedError


class Transform(Part):
    def forward(self, t: torch.Tensor, ctx) -> None:
        raise NotImplementedError
