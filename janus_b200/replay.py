"""Trace replay over the engine's step function (see `bin/trace_run`)."""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict



def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description="replay token ids step by step and write logits")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time, each rounded up to a multiple of 64")
    ap.add_argument("--no-graphs", action="store_true",
                    help="launch the kernels of single-token steps one by one instead of replaying them from "
                         "CUDA graphs, as generation does")
    args = ap.parse_args(argv)

    print("[trace_run] loading (kernels are compiled at the first call; this can take a minute)",
          file=sys.stderr, flush=True)
    import torch

    import janus_b200
    from janus_b200.cache import PAGE_SIZE
    from janus_b200.engine.step import StepEntry

    os.makedirs(args.out, exist_ok=True)
    # every live request holds at least one page: as many slots as pages serve any trace that
    # keeps within --max-tokens
    model = janus_b200.load(args.model, dtype=args.dtype, max_tokens=args.max_tokens,
                            max_slots=max(1, (args.max_tokens + PAGE_SIZE - 1) // PAGE_SIZE),
                            use_graphs=not args.no_graphs)
    slots: Dict[str, int] = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid = str(e["id"])
            if rid not in slots:
                slots[rid] = model.alloc_slot()
            entries.append(StepEntry(slots[rid], e["tokens"], e.get("want", [])))
        if entries:
            logits = model.step(entries)
            model.check()   # waits for the step; no file is written from a step whose kernel gave up
            if logits.shape[0] > 0:
                arr = logits.detach().to("cpu", torch.float32).numpy().astype("<f4", copy=False)
                tmp = os.path.join(args.out, f".{step}.f32.tmp")
                arr.tofile(tmp)
                os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
        for rid in rec.get("end", []):
            rid = str(rid)
            if rid in slots:
                model.free_slot(slots.pop(rid))
        print(f"done {step}", flush=True)
    return 0
