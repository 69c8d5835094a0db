"""A decoder built from a `ModelSpec`: embedding, layers made of registered
parts, the order in which they run, final norm and head.

The forward pass follows crates/janus-engine/src/model/transformer/forward.rs:25-119
(embed, blocks, final norm, head), but runs all tokens of a step at once and
computes logits only for the rows that are wanted.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import log
from ..kernels import ops
from ..parts.base import CacheSpec, LayerSpec, ModelSpec, make_part
from ..parts.linear import Linear
from ..weights.loader import TensorSpec, load_named


def _layer_parts(spec: LayerSpec):
    return spec.parts()


class DecoderModel:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device: torch.device):
        self.spec, self.dtype, self.device = spec, dtype, device
        self.hidden_size, self.vocab_size = spec.hidden_size, spec.vocab_size
        self.layers = []
        self._layer_part_objs: List[Dict[str, object]] = []
        for ls in spec.layers:
            objs = {attr: make_part(family, ps, dtype, device) for attr, family, ps in _layer_parts(ls)}
            self._layer_part_objs.append(objs)
            self.layers.append(_arrange(ls.arrangement, objs, spec.hidden_size, dtype))
        self.final_norm = make_part("norm", spec.final_norm, dtype, device)
        self.embedding_transforms = [make_part("transform", ps, dtype, device) for ps in spec.embedding_transforms]
        self.logit_transforms = [make_part("transform", ps, dtype, device) for ps in spec.logit_transforms]
        self.embedding: Optional[torch.Tensor] = None
        self.head = Linear(spec.hidden_size, spec.vocab_size, dtype, device, name="head")
        self.schedule = list(spec.schedule)
        for place, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule place {place} names layer {e.layer}, the model has {len(self.layers)}")
            if e.reads_cache_of is not None:
                if not 0 <= e.reads_cache_of < place or self.schedule[e.reads_cache_of].reads_cache_of is not None:
                    raise ValueError(f"schedule place {place} must read the cache of an earlier place that writes one")

    # -- what the cache must provide ----------------------------------------------
    def place_cache_specs(self) -> List[CacheSpec]:
        out: List[CacheSpec] = []
        for e in self.schedule:
            out.append(None if e.reads_cache_of is not None
                       else self._layer_part_objs[e.layer]["mixer"].cache_spec())
        return out

    def limit_positions(self, n: int) -> None:
        """The engine's longest sequence: parts that tabulate something per position
        (rotary tables) need no more rows than that."""
        for objs in self._layer_part_objs:
            for part in objs.values():
                limit = getattr(part, "limit_positions", None)
                if limit is not None:
                    limit(n)

    # -- weights --------------------------------------------------------------------
    def weight_specs(self) -> List[TensorSpec]:
        return model_weight_specs(self.spec, self._layer_part_objs, self.final_norm,
                                  self.embedding_transforms + self.logit_transforms)

    def load(self, checkpoint) -> None:
        spec = self.spec
        named = load_named(checkpoint, self.weight_specs(), ignorable=spec.ignorable_weights,
                           engine_dtype=self.dtype)
        emb = named[spec.embedding_weight]
        self.embedding = emb.to(device=self.device, dtype=self.dtype).contiguous()
        if spec.head_weight is None:
            self.head.load_row_major(self.embedding)
        else:
            self.head.load([named[spec.head_weight]])
        self.final_norm.load(**{k: named[v] for k, v in spec.final_norm.weights.items()})
        for ls, objs in zip(spec.layers, self._layer_part_objs):
            for attr, _family, ps in _layer_parts(ls):
                objs[attr].load(**{k: named[v] for k, v in ps.weights.items()})
        for ps, part in zip(spec.embedding_transforms + spec.logit_transforms,
                            self.embedding_transforms + self.logit_transforms):
            part.load(**{k: named[v] for k, v in ps.weights.items()})

    # -- forward ----------------------------------------------------------------------
    def forward(self, ctx, want_rows: torch.Tensor, logits: torch.Tensor) -> None:
        """Run the tokens of `ctx` through every place of the schedule and write
        the logits of the rows `want_rows` (indices into the step's tokens)."""
        with ops.stream_scope():         # every launch of the pass goes to the stream that is current now
            self._forward(ctx, want_rows, logits)

    def _forward(self, ctx, want_rows: torch.Tensor, logits: torch.Tensor) -> None:
        T = ctx.n_tokens
        residual = ctx.workspace.get("residual", (T, self.hidden_size), torch.float32)
        ops.embed_gather(self.embedding, ctx.token_ids, residual, ctx.feedback,
                         ctx.seq_slot if ctx.feedback is not None else None)
        for transform in self.embedding_transforms:
            transform.forward(residual, ctx)
        for place, entry in enumerate(self.schedule):
            view = ctx.cache_view(place if entry.reads_cache_of is None else entry.reads_cache_of)
            with log.nvtx_range(f"place {place}: layer {entry.layer}"):
                self.layers[entry.layer].forward(residual, ctx, view, writes_cache=entry.reads_cache_of is None)
        n_want = want_rows.shape[0]
        if n_want == 0:
            return
        z = ctx.workspace.get("final_normed", (n_want, self.hidden_size), self.dtype)
        self.final_norm.forward(residual, z, row_index=want_rows)
        self.head.forward(z, logits)
        for transform in self.logit_transforms:
            transform.forward(logits, ctx)


def _arrange(kind: str, objs: Dict[str, object], hidden_size: int, dtype: torch.dtype):
    from ..parts.base import _REGISTRIES
    try:
        factory = _REGISTRIES["arrangement"][kind]
    except KeyError:
        raise KeyError(f"no arrangement '{kind}' is registered") from None
    return factory(objs, hidden_size, dtype)


def model_weight_specs(spec: ModelSpec, layer_part_objs=None, final_norm=None, transforms=None) -> List[TensorSpec]:
    """Every tensor the model reads, with its shape, from the parts' own
    `weight_shapes()` and the spec's names.  Built on the CPU when no parts are
    given (the random-weights writer needs no device)."""
    cpu = torch.device("cpu")
    if layer_part_objs is None:
        layer_part_objs = [{attr: make_part(family, ps, torch.float32, cpu) for attr, family, ps in _layer_parts(ls)}
                           for ls in spec.layers]
        final_norm = make_part("norm", spec.final_norm, torch.float32, cpu)
        transforms = [make_part("transform", ps, torch.float32, cpu)
                      for ps in spec.embedding_transforms + spec.logit_transforms]
    out: Dict[str, TensorSpec] = {}

    def add(name: str, shape, init: str):
        prev = out.get(name)
        if prev is not None and tuple(prev.shape) != tuple(shape):
            raise ValueError(f"tensor '{name}' is wanted with shapes {prev.shape} and {tuple(shape)}")
        out[name] = TensorSpec(name, tuple(shape), init)

    add(spec.embedding_weight, (spec.vocab_size, spec.hidden_size), "normal")
    for ls, objs in zip(spec.layers, layer_part_objs):
        for attr, _family, ps in _layer_parts(ls):
            shapes = objs[attr].weight_shapes()
            if set(shapes) != set(ps.weights):
                raise ValueError(f"{ps.kind}: weights {sorted(shapes)} are needed, names are given for {sorted(ps.weights)}")
            for param, (shape, init) in shapes.items():
                add(ps.weights[param], shape, init)
    for param, (shape, init) in final_norm.weight_shapes().items():
        add(spec.final_norm.weights[param], shape, init)
    for ps, part in zip(spec.embedding_transforms + spec.logit_transforms, transforms or ()):
        shapes = part.weight_shapes()
        if set(shapes) != set(ps.weights):
            raise ValueError(f"{ps.kind}: weights {sorted(shapes)} are needed, names are given for {sorted(ps.weights)}")
        for param, (shape, init) in shapes.items():
            add(ps.weights[param], shape, init)
    if spec.head_weight is not None:
        add(spec.head_weight, (spec.vocab_size, spec.hidden_size), "normal")
    return list(out.values())
