"""Random-weights mode: a seeded checkpoint made from a configuration, and a
writer that turns it into a model folder (config.json + model.safetensors).

The reference has no such mode (its tests use zero or hand-made buffers).  The
generator is counter-based: element i of a tensor is a function of (seed, tensor
name, i) alone, so a tensor's values do not depend on which other tensors exist,
on the order of creation, or on the device that evaluates the function.  It uses
64-bit integer arithmetic and exact float operations only (no logarithm, no
cosine), so the host and the device give the same bits: a model made on the GPU
can be made again on the CPU for an oracle.
Matrices and embeddings are ~N(0, std); norm weights are 1 + ~N(0, norm_std).
The normal variate is the sum of twelve uniform 16-bit integers, centred and
scaled to variance one (Irwin-Hall: tails end at six standard deviations).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, List, Sequence, Tuple

import torch

from .loader import TensorSpec
from .safetensors_io import save_file

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32,
           "bf16": torch.bfloat16, "fp32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    try:
        return _DTYPES[name]
    except KeyError:
        raise ValueError(f"dtype must be 'bfloat16' or 'float32', got {name!r}") from None


_CHUNK = 1 << 24          # elements made at a time (bounds the int64 temporaries to a few hundred MB)
_GOLDEN = 0x9E3779B97F4A7C15
_MIX1 = 0xBF58476D1CE4E5B9
_MIX2 = 0x94D049BB133111EB
DRAWS = 3                 # 64-bit draws per element, four 16-bit uniforms each


def _signed(x: int) -> int:
    """A 64-bit pattern as the int64 that holds it."""
    x &= (1 << 64) - 1
    return x - (1 << 64) if x >= (1 << 63) else x


def tensor_key(seed: int, name: str) -> int:
    """64 bits from (seed, tensor name)."""
    digest = hashlib.sha256(f"{int(seed)}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little")


def _mix64(x: torch.Tensor) -> torch.Tensor:
    """The splitmix64 finaliser on int64 tensors (products wrap; shifts made logical by masks)."""
    x = (x ^ ((x >> 30) & ((1 << 34) - 1))) * _signed(_MIX1)
    x = (x ^ ((x >> 27) & ((1 << 37) - 1))) * _signed(_MIX2)
    return x ^ ((x >> 31) & ((1 << 33) - 1))


def standard_normal(key: int, start: int, count: int, device) -> torch.Tensor:
    """Elements [start, start + count) of the stream `key`, float32: for element i the draws
    mix64(key + (DRAWS * i + d + 1) * golden), d = 0..2, each cut into four 16-bit integers; their sum,
    less its mean 12 * 65535 / 2, times 2^-16.  Every operation is exact in both int64 and float32, so
    the CPU and a CUDA device give the same bits."""
    i = torch.arange(start, start + count, dtype=torch.int64, device=device)
    total = torch.zeros(count, dtype=torch.int64, device=device)
    for d in range(DRAWS):
        h = _mix64((i * DRAWS + (d + 1)) * _signed(_GOLDEN) + _signed(key))
        total += (h & 0xFFFF) + ((h >> 16) & 0xFFFF) + ((h >> 32) & 0xFFFF) + ((h >> 48) & 0xFFFF)
    return (total - 6 * 65535).to(torch.float32) * (1.0 / 65536.0)


class RandomCheckpoint:
    """Checkpoint interface (`names, shape, dtype, tensor`) over seeded noise."""

    def __init__(self, specs: Sequence[TensorSpec], seed: int, dtype="bfloat16",
                 std: float = 0.02, norm_std: float = 0.02, device: str = "cpu"):
        self._specs: Dict[str, TensorSpec] = {s.name: s for s in specs if not s.optional}
        self.seed = int(seed)
        self._dtype = parse_dtype(dtype)
        self.std = float(std)
        self.norm_std = float(norm_std)
        self.device = torch.device(device)

    def names(self) -> List[str]:
        return list(self._specs)

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(self._specs[name].shape)

    def dtype(self, name: str) -> torch.dtype:
        return self._dtype

    def tensor(self, name: str) -> torch.Tensor:
        spec = self._specs[name]
        n = 1
        for d in spec.shape:
            n *= int(d)
        out = torch.empty(n, dtype=self._dtype, device=self.device)
        key = tensor_key(self.seed, name)
        for start in range(0, n, _CHUNK):
            z = standard_normal(key, start, min(_CHUNK, n - start), self.device)
            if spec.init == "ones":
                z = z * self.norm_std + 1.0
            else:
                z = z * self.std
            out[start:start + z.numel()] = z.to(self._dtype)
        return out.view(tuple(spec.shape))


def write_random_model(config_dict: dict, out_dir: str, seed: int, dtype="bfloat16",
                       std: float = 0.02, norm_std: float = 0.02) -> str:
    """Write `out_dir/config.json` and `out_dir/model.safetensors` for the
    architecture that `config_dict` names.  Returns `out_dir`."""
    from ..config.registry import resolve_architecture

    arch = resolve_architecture(config_dict)
    config = arch.config_class.from_dict(config_dict)
    specs = arch.weight_specs(config)
    ck = RandomCheckpoint(specs, seed, dtype=dtype, std=std, norm_std=norm_std)
    os.makedirs(out_dir, exist_ok=True)
    out_cfg = config.to_dict()
    out_cfg["torch_dtype"] = "bfloat16" if parse_dtype(dtype) == torch.bfloat16 else "float32"
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(out_cfg, f, indent=2)
    save_file({n: ck.tensor(n) for n in ck.names()}, os.path.join(out_dir, "model.safetensors"),
              metadata={"format": "pt", "seed": str(seed)})
    return out_dir
