"""Weights by tensor name.

A checkpoint is anything with `names()`, `shape(name)`, `dtype(name)` and
`tensor(name)`: a model folder's safetensors file(s) or a seeded random source.
`load_named` hands a model the tensors it asks for and raises ONE error that
lists every missing tensor, every unexpected tensor and every wrong shape,
before anything is copied to a device.  (The reference reports one missing name
at a time, crates/janus-engine/src/model/block.rs:19-51, and only warns on a
size mismatch, crates/janus-engine/src/formats/safetensors.rs:137-146.)

Stored dtypes are kept for the bfloat16 engine: 16-bit floats become bfloat16
(float16 is rounded once, to nearest even), a tensor stored in 32-bit floats
stays float32, integer tables become int32.  The float32 engine widens every
stored float exactly (the reference widens each stored dtype before its one
rounding, crates/janus-engine/src/compute/engine.rs:446-633); float16 is never
rounded to bfloat16 on the way.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Dict, Iterable, List, Sequence, Tuple

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile


class WeightError(ValueError):
    """Tensors of a checkpoint do not fit the model."""


@dataclass(frozen=True)
class TensorSpec:
    """What a model expects of one tensor.  `init` tells the random source how
    to fill it: "normal" (N(0, std)) or "ones" (1 + N(0, norm_std))."""
    name: str
    shape: Tuple[int, ...]
    init: str = "normal"
    optional: bool = False


class FolderCheckpoint:
    """`model.safetensors`, or the shards named by `model.safetensors.index.json`
    (the reference reads the single file, crates/janus-engine/examples/inference.rs:118-122)."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        index = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        self._where: Dict[str, SafetensorsFile] = {}
        if os.path.exists(single):
            files = [single]
        elif os.path.exists(index):
            try:
                with open(index) as f:
                    weight_map = json.load(f)["weight_map"]
                files = sorted({os.path.join(model_dir, v) for v in weight_map.values()})
            except (OSError, ValueError, KeyError, TypeError, AttributeError) as e:
                raise WeightError(f"'{index}' is no shard index (a JSON object with a 'weight_map' of tensor "
                                  f"name -> file name): {e!r}") from e
        else:
            raise WeightError(
                f"no weights in '{model_dir}': expected model.safetensors or model.safetensors.index.json")
        for path in files:
            try:
                sf = SafetensorsFile(path)
            except SafetensorsError as e:
                raise WeightError(str(e)) from e
            for n in sf.names():
                if n in self._where:
                    raise WeightError(f"tensor '{n}' is stored twice: in '{self._where[n].path}' and in '{path}'")
                self._where[n] = sf

    def names(self) -> List[str]:
        return list(self._where)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self._where[name].shape(name)

    def dtype(self, name: str) -> torch.dtype:
        return self._where[name].dtype(name)

    def tensor(self, name: str) -> torch.Tensor:
        return self._where[name].tensor(name)


def kept_dtype(stored: torch.dtype, engine_dtype: torch.dtype = torch.bfloat16) -> torch.dtype:
    """The dtype a stored tensor is handed out in, for an engine of `engine_dtype`."""
    if stored in (torch.bfloat16, torch.float16):
        return torch.float32 if engine_dtype == torch.float32 else torch.bfloat16
    if stored in (torch.float32, torch.float64):
        return torch.float32
    if stored in (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8, torch.bool):
        return torch.int32
    raise WeightError(f"unsupported stored dtype {stored}")


def check_names(checkpoint, specs: Sequence[TensorSpec], ignorable: Iterable[str] = ()) -> None:
    """Raise one WeightError naming all misfits; return silently if none."""
    have = set(checkpoint.names())
    wanted = {s.name for s in specs}
    missing = [s.name for s in specs if s.name not in have and not s.optional]
    unexpected = sorted(have - wanted - set(ignorable))
    wrong = []
    for s in specs:
        if s.name in have and tuple(checkpoint.shape(s.name)) != tuple(s.shape):
            wrong.append(f"{s.name}: expected {list(s.shape)}, got {list(checkpoint.shape(s.name))}")
    if not (missing or unexpected or wrong):
        return
    parts = ["checkpoint does not fit the model:"]
    if missing:
        parts.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        parts.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong:
        parts.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(wrong))
    raise WeightError("\n".join(parts))


class NamedTensors:
    """Lazy mapping name -> tensor in its kept dtype; a tensor is fetched from
    the checkpoint when a part asks for it, so a model larger than host memory
    can still be placed tensor by tensor."""

    def __init__(self, checkpoint, names: Iterable[str], engine_dtype: torch.dtype = torch.bfloat16):
        self._checkpoint = checkpoint
        self._names = set(names)
        self._engine_dtype = engine_dtype

    def __contains__(self, name: str) -> bool:
        return name in self._names

    def __getitem__(self, name: str) -> torch.Tensor:
        if name not in self._names:
            raise KeyError(name)
        t = self._checkpoint.tensor(name)
        return t.to(kept_dtype(t.dtype, self._engine_dtype))

    def keys(self):
        return sorted(self._names)


def load_named(checkpoint, specs: Sequence[TensorSpec], ignorable: Iterable[str] = (),
               engine_dtype: torch.dtype = torch.bfloat16) -> NamedTensors:
    """Check the whole checkpoint against the specs (one error for all
    misfits), then give access to the tensors the specs name, in the dtype
    an engine of `engine_dtype` keeps them in."""
    check_names(checkpoint, specs, ignorable)
    have = set(checkpoint.names())
    return NamedTensors(checkpoint, [s.name for s in specs if s.name in have], engine_dtype)
