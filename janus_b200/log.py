"""Logging to stderr by level, set with JANUS_LOG=error|warn|info|debug (default: warn), and NVTX ranges
around the phases of a step with JANUS_NVTX=1.  The reference logs through `tracing` macros with a `fmt`
subscriber (crates/janus-engine/examples/inference.rs:96) and prints its telemetry block after a generation
(crates/janus-engine/src/model/transformer/generation.rs:295-307)."""
from __future__ import annotations

import contextlib
import os
import sys

LEVELS = {"error": 0, "warn": 1, "info": 2, "debug": 3}


def parse_level(text) -> int:
    """`JANUS_LOG`'s value as a number; unknown words fall back to "warn"."""
    return LEVELS.get(str(text or "warn").strip().lower(), LEVELS["warn"])


_level = [parse_level(os.environ.get("JANUS_LOG"))]
_nvtx = [os.environ.get("JANUS_NVTX", "0") == "1"]


def set_level(name: str) -> None:
    _level[0] = parse_level(name)


def enabled(name: str) -> bool:
    return LEVELS[name] <= _level[0]


def log(name: str, message: str) -> None:
    if LEVELS[name] <= _level[0]:
        print(f"[janus_b200 {name}] {message}", file=sys.stderr, flush=True)


@contextlib.contextmanager
def nvtx_range(label: str):
    """An NVTX range on the calling thread (a profiler's timeline shows it over the kernels launched inside);
    nothing unless JANUS_NVTX=1."""
    if not _nvtx[0]:
        yield
        return
    import torch
    torch.cuda.nvtx.range_push(label)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()
