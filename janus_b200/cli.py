"""Command line in the manner of the reference's examples: a model folder in,
tokens out.

    python -m janus_b200 <model_dir> "<prompt>" ["<prompt>" ...] [--batch-size N] [--max-tokens N] [--temperature T]

Positional `<model_dir> "<prompt>"` as crates/janus-engine/examples/inference.rs:102-133
(the folder holds config.json and model.safetensors, inference.rs:118-125);
`--batch-size`, `--max-tokens`, `--temperature` with the meanings and defaults
of crates/janus-engine/examples/batch_inference.rs:101-147 (4, 50, 0.0 = greedy).
The reference's tokenizer reads only GGUF metadata and is out of scope here, so a
prompt is a list of token ids ("1,15043,3186" or "1 15043 3186").  The remaining
options carry the sampler's names (crates/janus-engine/src/model/sampler.rs:20-39).
Longer spellings are accepted for the same options (`--prompt-ids`, `--prompt-ids-file`,
`--max-new-tokens`, `--max-batch`, `--max-seq-len`, `--dtype bf16|fp32`), and
`--random-weights [--seed-weights S]` runs a folder that holds only config.json.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List


def parse_prompt(text: str) -> List[int]:
    try:
        ids = [int(t) for t in text.replace(",", " ").split()]
    except ValueError:
        raise SystemExit(f"Error: a prompt is a list of token ids, got '{text}'") from None
    if not ids:
        raise SystemExit("Error: empty prompt")
    return ids


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(
        prog="janus_b200",
        usage='%(prog)s <model_dir> "<prompt>" [--batch-size N] [--max-tokens N] [--temperature T]')
    ap.add_argument("model_dir", help="folder with config.json and model.safetensors")
    ap.add_argument("prompts", nargs="*", help='token ids of a prompt, e.g. "1,2,3"; several prompts form a batch')
    ap.add_argument("--prompt-ids", action="append", default=[], help="a prompt as an option (repeatable)")
    ap.add_argument("--prompts-file", "--prompt-ids-file", action="append", default=[],
                    help="file with one prompt (token ids) per line (repeatable)")
    ap.add_argument("--batch-size", "--max-batch", type=int, default=4,
                    help="prompts processed in parallel (default: 4)")
    ap.add_argument("--max-tokens", "--max-new-tokens", type=int, default=50,
                    help="tokens to generate per sequence at most (default: 50)")
    ap.add_argument("--temperature", type=float, default=0.0, help="sampling temperature (default: 0.0 = greedy)")
    ap.add_argument("--top-k", type=int, default=0, help="top-k filtering (0 = disabled)")
    ap.add_argument("--top-p", type=float, default=1.0, help="top-p (nucleus) filtering (1.0 = disabled)")
    ap.add_argument("--repetition-penalty", type=float, default=1.0, help="repetition penalty (1.0 = none)")
    ap.add_argument("--seed", type=int, default=0, help="seed of the sampler's random numbers")
    ap.add_argument("--stop-id", type=int, action="append", default=[], help="extra stop token id (repeatable)")
    ap.add_argument("--ignore-eos", action="store_true", help="do not stop at config.json's eos_token_id")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "bf16", "fp32"])
    ap.add_argument("--context-size", "--max-seq-len", type=int, default=None,
                    help="longest sequence (default: the model's)")
    ap.add_argument("--max-step-tokens", type=int, default=32768,
                    help="prompts of a batch run in steps of at most this many tokens (default: 32768; 0 = one step)")
    ap.add_argument("--random-weights", action="store_true",
                    help="the folder holds only config.json: run it with random weights")
    ap.add_argument("--seed-weights", type=int, default=0, help="seed of --random-weights")
    ap.add_argument("--json", action="store_true", help="print one JSON object instead of text")
    ap.add_argument("--profile", metavar="FILE", default=None,
                    help="after generating, time the kernels of the first batch's prompt step and of one decode "
                         "step one by one and write them to FILE as JSON")
    args = ap.parse_args(argv)

    prompts = [parse_prompt(p) for p in list(args.prompts) + args.prompt_ids]
    for path in args.prompts_file:
        with open(path) as f:
            prompts += [parse_prompt(line) for line in f if line.strip()]
    if not prompts:
        ap.error("give at least one prompt")

    import janus_b200
    from janus_b200.engine.generate import tokens_held

    batch = max(1, min(args.batch_size, len(prompts)))
    room = sorted((tokens_held(len(p), args.max_tokens, 64) for p in prompts), reverse=True)
    dtype = {"bf16": "bfloat16", "fp32": "float32"}.get(args.dtype, args.dtype)
    if args.random_weights:
        with open(os.path.join(args.model_dir, "config.json")) as f:
            config = json.load(f)
        model = janus_b200.load_random(config, seed=args.seed_weights, dtype=dtype, max_tokens=sum(room[:batch]),
                                       max_seq_len=args.context_size, max_slots=batch,
                                       max_step_tokens=args.max_step_tokens or None)
    else:
        model = janus_b200.load(args.model_dir, dtype=dtype, max_tokens=sum(room[:batch]),
                                max_seq_len=args.context_size, max_slots=batch,
                                max_step_tokens=args.max_step_tokens or None)
    out, reasons, stats = model.generate(
        prompts, max_tokens=args.max_tokens, temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
        repetition_penalty=args.repetition_penalty, seed=args.seed, stop_token_ids=args.stop_id,
        ignore_eos=args.ignore_eos, batch_size=batch, return_reasons=True)
    if args.profile:
        with open(args.profile, "w") as f:
            json.dump(model.profile(prompts[:batch]), f, indent=1)
    if args.json:
        print(json.dumps({"tokens": out, "finish_reasons": reasons, "prefill_tokens_per_s": stats.prefill_tokens_per_s,
                          "decode_tokens_per_s": stats.decode_tokens_per_s, "graph_captures": stats.graph_captures}))
        return 0
    print("=== janus_b200 inference ===")
    print(f"Batch size: {batch}\nMax tokens per sequence: {args.max_tokens}\nTemperature: {args.temperature}\n")
    for i, (p, o, r) in enumerate(zip(prompts, out, reasons)):
        print(f"[{i}] prompt ({len(p)} tokens) -> {len(o)} tokens, finish reason: {r}")
        print("    " + " ".join(map(str, o)))
    print(f"\nPrefill: {stats.prefill_tokens} tokens in {stats.prefill_ms:.1f} ms ({stats.prefill_tokens_per_s:.0f} tok/s)")
    print(f"Decode:  {stats.decode_tokens} tokens in {stats.decode_ms:.1f} ms ({stats.decode_tokens_per_s:.0f} tok/s, "
          f"{stats.decode_steps} steps, {stats.batches} batches, {stats.graph_captures} decode graphs recorded)")
    return 0


def run(argv=None) -> int:
    """`main` for a person at a terminal: what the library refuses (a bad config.json, missing or misshapen
    tensors, a prompt outside the vocabulary or longer than the cache, a size the kernels do not take) is one
    line on stderr and exit code 1, not a traceback (JANUS_LOG=debug keeps the traceback)."""
    from . import log
    from .cache.pages import CacheFull
    from .config.base import ConfigError
    from .engine.step import StepError
    from .kernels.build import KernelBuildError
    from .kernels.ops import KernelError
    from .weights.loader import WeightError
    from .weights.safetensors_io import SafetensorsError
    try:
        return main(argv)
    except (ConfigError, WeightError, SafetensorsError, StepError, CacheFull, KernelError, KernelBuildError,
            FileNotFoundError, ValueError) as e:
        if log.enabled("debug"):
            raise
        print(f"Error: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(run())
