"""Shared pieces of the tests: the two tiny configurations, model folders with
random weights, the replay driver and the comparison rule.

Tolerances are fixed here once: the largest difference of two logit arrays,
divided by the largest reference logit, must stay below FP32_TOL when the engine
runs in float32 and below BF16_TOL when it runs in bfloat16.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
from typing import Dict, List, Sequence

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

FP32_TOL = 1e-4
BF16_TOL = 3e-2

# Two configurations that differ in every size and option.
TINY_A = dict(
    architectures=["LlamaForCausalLM"], hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
    num_key_value_heads=2, intermediate_size=192, vocab_size=256, max_position_embeddings=128,
    rms_norm_eps=1e-5, rope_theta=10000.0, rope_scaling=None, tie_word_embeddings=False,
    eos_token_id=[250, 251])
TINY_B = dict(
    architectures=["LlamaForCausalLM"], hidden_size=96, num_hidden_layers=3, num_attention_heads=3,
    num_key_value_heads=1, head_dim=40, intermediate_size=320, vocab_size=384, max_position_embeddings=256,
    rms_norm_eps=1e-6, rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=4.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=32),
    tie_word_embeddings=True, eos_token_id=383)
TINY = {"A": TINY_A, "B": TINY_B}


def make_model_dir(cfg: dict, out_dir: str, seed: int, dtype: str, sharpen: float = 6.0,
                   stored: str = None, shards: int = 1) -> str:
    """A model folder with random weights; q and k projections are scaled by
    `sharpen` so that attention is peaked and a wrong key shows in the logits.
    `stored`: "float16" writes the file in float16 (values made in float32);
    `shards` > 1 writes that many files and `model.safetensors.index.json`."""
    from janus_b200.config import resolve_architecture
    from janus_b200.weights import RandomCheckpoint, save_file

    arch = resolve_architecture(cfg)
    config = arch.config_class.from_dict(cfg)
    # the random source gives the same bits on every device: a GPU, where there is one, is only faster
    device = "cuda" if torch.cuda.is_available() else "cpu"
    ck = RandomCheckpoint(arch.weight_specs(config), seed, dtype="float32" if stored else dtype, std=0.02,
                          norm_std=0.02, device=device)
    tensors = {}
    for name in ck.names():
        t = ck.tensor(name).cpu()
        if name.endswith("q_proj.weight") or name.endswith("k_proj.weight"):
            t = (t.float() * sharpen).to(t.dtype)
        if stored:
            t = t.to(getattr(torch, stored))
        tensors[name] = t
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg, f)
    if shards <= 1:
        save_file(tensors, os.path.join(out_dir, "model.safetensors"))
        return out_dir
    names = sorted(tensors)
    weight_map = {}
    for i in range(shards):
        fname = f"model-{i + 1:05d}-of-{shards:05d}.safetensors"
        mine = names[i::shards]
        save_file({n: tensors[n] for n in mine}, os.path.join(out_dir, fname))
        weight_map.update({n: fname for n in mine})
    with open(os.path.join(out_dir, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f)
    return out_dir


def random_tokens(n: int, vocab: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def rel_err(got, ref) -> float:
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, f"shape {got.shape} != {ref.shape}"
    assert np.isfinite(got).all(), "non-finite values in the engine's output"
    return float(np.abs(got - ref).max() / (np.abs(ref).max() + 1e-12))


def tol_for(dtype: str) -> float:
    return FP32_TOL if dtype == "float32" else BF16_TOL


class TraceRun:
    """Drives `bin/trace_run` as a user does: steps in on stdin, one at a time
    after the `done` line of the one before; logits back from files."""

    def __init__(self, model_dir: str, dtype: str, out_dir: str, max_tokens: int, graphs: bool = True):
        self.out_dir = out_dir
        env = dict(os.environ)
        self.proc = subprocess.Popen(
            [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
             "--out", out_dir, "--max-tokens", str(max_tokens)] + ([] if graphs else ["--no-graphs"]),
            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
        self.step_no = 0

    def step(self, entries: Sequence[dict], end: Sequence[str] = ()) -> np.ndarray:
        n = self.step_no
        self.step_no += 1
        self.proc.stdin.write(json.dumps({"step": n, "entries": list(entries), "end": list(end)}) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline()
        if line.strip() != f"done {n}":
            rest = self.proc.stdout.read()
            raise RuntimeError(f"trace_run answered {line!r} {rest!r} to step {n} (exit {self.proc.poll()})")
        wanted = sum(len(e.get("want", [])) for e in entries)
        path = os.path.join(self.out_dir, f"{n}.f32")
        if wanted == 0:
            assert not os.path.exists(path)
            return np.zeros((0, 0), dtype=np.float32)
        return np.fromfile(path, dtype="<f4").reshape(wanted, -1)

    def close(self) -> int:
        self.proc.stdin.close()
        code = self.proc.wait(timeout=120)
        return code
