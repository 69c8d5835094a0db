"""Random-weights mode: a seeded checkpoint made from a configuration, and a
writer that turns it into a model folder (config.json + model.safetensors).

The reference has no such mode (its tests use zero or hand-made buffers).  Each
tensor has a generator of its own, keyed by (seed, tensor name), so a tensor's
values do not depend on which other tensors exist or on the order of creation.
Matrices and embeddings are N(0, std); norm weights are 1 + N(0, norm_std).
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

    def _generator(self, name: str) -> torch.Generator:
        digest = hashlib.sha256(f"{self.seed}:{name}".encode()).digest()
        g = torch.Generator(device=self.device)
        g.manual_seed(int.from_bytes(digest[:8], "little") & ((1 << 63) - 1))
        return g

    def tensor(self, name: str) -> torch.Tensor:
        spec = self._specs[name]
        g = self._generator(name)
        x = torch.randn(spec.shape, generator=g, dtype=torch.float32, device=self.device)
        if spec.init == "ones":
            x = 1.0 + self.norm_std * x
        else:
            x = self.std * x
        return x.to(self._dtype)


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
