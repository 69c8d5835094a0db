"""The Python entry point: a model folder in, tokens out.

The reference has no `Model::from_dir`; each of its examples loads by hand
(crates/janus-engine/examples/inference.rs:199-309: config, safetensors, blocks,
sampler, `Model::new`, `generate`).  `load` does the same steps here, choosing
the model class by config.json's `architectures`.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import numpy as np
import torch

from . import log
from .cache import PAGE_SIZE
from .config import read_config_json, resolve_architecture
from .engine.generate import plan_prompt_steps, run_generation
from .engine.step import Engine, EngineOptions, StepEntry
from .sampling import DeviceSampler, SamplerConfig
from .weights import FolderCheckpoint, RandomCheckpoint, parse_dtype


class _EngineBackend:
    """Drives the engine's step function and the device sampler for the
    generation loop."""

    def __init__(self, engine: Engine, sampler: DeviceSampler):
        self.engine, self.sampler = engine, sampler
        self.device = engine.device
        self._staging = None      # pinned buffers the sampled tokens are copied into
        self._turn = 0
        if not engine.options.use_graphs:
            self.decode_launch = None   # no device-side token feedback without graphs: plain loop

    def alloc_slot(self) -> int:
        slot = self.engine.alloc_slot()
        self.sampler.reset_row(slot)
        return slot

    def free_slot(self, slot: int) -> None:
        self.engine.free_slot(slot)

    def synchronize(self) -> None:
        torch.cuda.synchronize(self.device)

    def _sample(self, logits: torch.Tensor, slots, requests, steps) -> List[int]:
        meta = torch.tensor([list(requests), list(steps), list(slots)], dtype=torch.int32).to(self.device)
        ids = self.sampler.sample(logits, meta[0], meta[1], meta[2])
        return ids.cpu().tolist()

    def prefill(self, slots, prompts, requests) -> List[int]:
        steps = plan_prompt_steps([len(p) for p in prompts], self.engine.options.max_step_tokens)
        rows = None      # the logits at each prompt's last token, copied from the step that held it
        for pieces in steps:
            logits = self.engine.step([StepEntry(slots[i], prompts[i][a:b], (b - a - 1,) if b == len(prompts[i]) else ())
                                       for i, a, b in pieces])
            if len(steps) == 1:
                return self._sample(logits, slots, requests, [0] * len(slots))
            if rows is None:
                rows = torch.empty((len(prompts), logits.shape[1]), dtype=logits.dtype, device=logits.device)
            done = [i for i, _, b in pieces if b == len(prompts[i])]
            for row, i in enumerate(done):
                rows[i].copy_(logits[row])       # a device copy; the sampler reads all prompts' rows at once
        return self._sample(rows, slots, requests, [0] * len(slots))

    def decode(self, slots, last_tokens, requests, steps) -> List[int]:
        ids = self.engine.decode_sample(slots, last_tokens, self.sampler, requests, steps)
        return ids.cpu().tolist()

    # A step is launched and its tokens are fetched later, so that the host can lay
    # out the next step while the device runs this one.  A token -1 stands for the
    # one the step before sampled for that slot (it is read on the device).
    def decode_launch(self, slots, tokens, requests, steps):
        ids = self.engine.decode_sample(slots, tokens, self.sampler, requests, steps)
        if self._staging is None:
            self._staging = [torch.zeros(self.engine.cache.n_slots, dtype=torch.int32, pin_memory=True)
                             for _ in range(3)]
        buf = self._staging[self._turn % 3][:len(slots)]
        self._turn += 1
        buf.copy_(ids, non_blocking=True)       # ordered after the step, before the next one overwrites `ids`
        done = torch.cuda.Event()
        done.record()
        return buf, done

    def decode_collect(self, handle) -> List[int]:
        buf, done = handle
        done.synchronize()
        return buf.tolist()


class Model:
    """A loaded model with its cache and step function."""

    def __init__(self, config, engine: Engine):
        self.config = config
        self.engine = engine
        self.device = engine.device
        self.dtype = engine.dtype
        self._samplers = {}

    # -- the step function, for callers that schedule themselves ---------------
    def alloc_slot(self) -> int:
        return self.engine.alloc_slot()

    def free_slot(self, slot: int) -> None:
        self.engine.free_slot(slot)

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        return self.engine.step(entries)

    def profile(self, prompts: Sequence[Sequence[int]]) -> dict:
        """Where a step's time goes: the prompts' step and one decode step after it, each with its kernels
        launched one by one and timed by CUDA events (`Engine.profile_step`).  Takes and gives back one slot a
        prompt.  Returns {"prefill": {...}, "decode": {...}} with a row per kernel face: launches and
        milliseconds.  Decode steps of `generate` replay the same kernels from a CUDA graph, a little faster."""
        slots = [self.alloc_slot() for _ in prompts]
        try:
            prefill = self.engine.profile_step([StepEntry(s, [int(t) for t in p], (len(p) - 1,))
                                                for s, p in zip(slots, prompts)])
            decode = self.engine.profile_step([StepEntry(s, (int(p[-1]),), (0,)) for s, p in zip(slots, prompts)])
        finally:
            for s in slots:
                self.free_slot(s)
        self.check()
        return {"prefill": prefill, "decode": decode,
                "how": "kernels launched one by one; a kernel's time is the time between the events after the "
                       "launch before it and after its own on the stream"}

    def check(self) -> None:
        """Waits for the device and raises if a tensor-core kernel gave up on a wait (its result would
        be incomplete).  `generate` calls it before it returns; a caller of `step` calls it when it
        reads results."""
        from .kernels import ops
        ops.check_kernel_status(self.device)

    # -- generation ------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]], max_tokens: int = 128, temperature: float = 0.0,
                 top_k: int = 0, top_p: float = 1.0, repetition_penalty: float = 1.0, seed: int = 0,
                 stop_token_ids: Optional[Sequence[int]] = None, ignore_eos: bool = False,
                 batch_size: Optional[int] = None,
                 callback: Optional[Callable[[int, int], bool]] = None,
                 return_reasons: bool = False):
        """Generate up to `max_tokens` new tokens for each prompt (lists of token
        ids).  Stop tokens are the configuration's (config.json's
        `eos_token_id`) plus `stop_token_ids`, unless `ignore_eos`.  Returns (tokens, stats), or
        (tokens, reasons, stats) with `return_reasons`."""
        sc = SamplerConfig(temperature=temperature, top_k=top_k, top_p=top_p,
                           repetition_penalty=repetition_penalty, max_tokens=max_tokens)
        cache = self.engine.cache
        # samplers are kept: one with a repetition penalty owns a count table, and a decode
        # graph that was captured with it stays valid for the next call
        skey = (sc.temperature, sc.top_k, sc.top_p, sc.repetition_penalty, seed)
        sampler = self._samplers.get(skey)
        if sampler is None:
            if len(self._samplers) >= 8:
                self._samplers.clear()
            sampler = DeviceSampler(sc, self.engine.model.vocab_size, cache.n_slots, seed, self.device)
            self._samplers[skey] = sampler
        if ignore_eos:
            stop = []
        elif hasattr(self.config, "stop_token_ids"):
            stop = list(self.config.stop_token_ids())
        else:
            stop = list(getattr(self.config, "eos_token_id", ()) or ())
        stop += list(stop_token_ids or ())
        # room that is free now: a caller of alloc_slot/step may hold pages of its own
        free_tokens = min((g.pool.n_free for g in cache.groups), default=cache.n_pages) * PAGE_SIZE
        captures_before = self.engine.graph_captures
        outputs, reasons, stats = run_generation(
            _EngineBackend(self.engine, sampler), [np.asarray(p, dtype=np.int64).reshape(-1) for p in prompts],
            max_tokens, stop,
            batch_size or cache.n_slots, free_tokens, self.engine.max_seq_len,
            cache.n_free_slots, PAGE_SIZE, callback)
        stats.graph_captures = self.engine.graph_captures - captures_before
        self.check()
        log.log("info", f"generate: {stats.requests} requests in {stats.batches} batches; prefill {stats.prefill_tokens} "
                        f"tokens at {stats.prefill_tokens_per_s:.0f} tok/s; decode {stats.decode_tokens} tokens in "
                        f"{stats.decode_steps} steps at {stats.decode_tokens_per_s:.0f} tok/s; "
                        f"{stats.graph_captures} decode graphs recorded")
        if return_reasons:
            return outputs, reasons, stats
        return outputs, stats


_WHOLE = object()        # max_step_tokens left at the engine's default


def _build(config_dict: dict, checkpoint_factory, dtype, max_tokens: int, max_seq_len: Optional[int],
           max_slots: Optional[int], device, use_graphs: bool, max_step_tokens=_WHOLE) -> Model:
    if not torch.cuda.is_available():
        raise RuntimeError("janus_b200 needs a CUDA device (sm_100a); there is no CPU path")
    device = torch.device(device)
    from .kernels import ops
    ops.bind_device(device)
    torch_dtype = parse_dtype(dtype)
    arch = resolve_architecture(config_dict)
    config = arch.config_class.from_dict(config_dict)
    with torch.cuda.device(device):
        model = arch.build(config, torch_dtype, device)
        model.load(checkpoint_factory(arch, config))
        options = EngineOptions(max_tokens=max_tokens, max_seq_len=max_seq_len, max_slots=max_slots,
                                use_graphs=use_graphs)
        if max_step_tokens is not _WHOLE:
            options.max_step_tokens = max_step_tokens
        engine = Engine(model, options)
    if log.enabled("info"):
        cache = engine.cache
        log.log("info", f"loaded {type(config).__name__}: {len(model.layers)} layers, hidden {model.hidden_size}, "
                        f"vocabulary {model.vocab_size}, dtype {torch_dtype}; cache of {cache.n_pages} pages of "
                        f"{PAGE_SIZE} tokens in {len(cache.groups)} group(s), {cache.n_slots} slots, longest sequence "
                        f"{engine.max_seq_len}; CUDA graphs {'on' if use_graphs else 'off'}")
    return Model(config, engine)


def load(model_dir: str, dtype="bfloat16", max_tokens: int = 8192, max_seq_len: Optional[int] = None,
         max_slots: Optional[int] = None, device="cuda:0", use_graphs: bool = True,
         max_step_tokens=_WHOLE) -> Model:
    """Load `model_dir` (config.json + model.safetensors).  `dtype` is the engine
    dtype: "bfloat16" (tensor-core kernels) or "float32" (true 32-bit path).
    `max_tokens` sizes the cache: the most tokens live sequences hold at any
    time, each sequence rounded up to a multiple of 64.  `max_step_tokens`: `generate` cuts a batch's
    prompts into steps of at most that many tokens (default 32,768; None: one step whatever the size)."""
    return _build(read_config_json(model_dir), lambda arch, config: FolderCheckpoint(model_dir), dtype,
                  max_tokens, max_seq_len, max_slots, device, use_graphs, max_step_tokens)


def load_random(config_dict: dict, seed: int, dtype="bfloat16", max_tokens: int = 8192,
                max_seq_len: Optional[int] = None, max_slots: Optional[int] = None, device="cuda:0",
                std: float = 0.02, norm_std: float = 0.0, use_graphs: bool = True,
                stored_dtype=None, max_step_tokens=_WHOLE) -> Model:
    """A model with seeded random weights made on the device, without a folder.  `stored_dtype` is the
    dtype the weights are "stored" in (default: the engine dtype): "bfloat16" under a float32 engine gives
    the 32-bit engine exactly the weights that the bfloat16 engine has.  The values are a function of the
    seed and the tensor's name alone, the same on every device (`weights.RandomCheckpoint`)."""
    def factory(arch, config):
        return RandomCheckpoint(arch.weight_specs(config), seed, dtype=stored_dtype or dtype, std=std,
                                norm_std=norm_std, device=device)
    return _build(config_dict, factory, dtype, max_tokens, max_seq_len, max_slots, device, use_graphs,
                  max_step_tokens)
