"""The generation loop: batches of unequal prompts, one prefill step per batch,
then one token per live sequence per step; sequences that meet a stop token or
their budget leave the batch at once and give their slot back; batches follow
one another until every request is served.

The loop's decisions are plain Python over a small backend interface, so they
can be tested without a device.  Compared with the reference's `generate_batch`
(crates/janus-engine/src/model/transformer/generation.rs:673-876): prompts are
not padded (728-738), finished rows do not stay in the batch (810-832), and the
stop token is not part of the output (as in `generate`, 241-263).  Finish
reasons are "stop" and "length" (generation.rs:421-427).
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Callable, List, Optional, Protocol, Sequence, Tuple


class GenerationBackend(Protocol):
    def alloc_slot(self) -> int: ...
    def free_slot(self, slot: int) -> None: ...
    def prefill(self, slots: Sequence[int], prompts: Sequence[Sequence[int]],
                requests: Sequence[int]) -> List[int]:
        """Run whole prompts in one step; return the first new token of each."""
    def decode(self, slots: Sequence[int], last_tokens: Sequence[int], requests: Sequence[int],
               steps: Sequence[int]) -> List[int]:
        """Run one token per sequence; return the next token of each.
        `steps[i]` is the number of tokens request i has produced so far."""
    def synchronize(self) -> None: ...


@dataclass
class GenerationStats:
    requests: int = 0
    batches: int = 0
    prefill_tokens: int = 0
    prefill_ms: float = 0.0
    decode_steps: int = 0
    decode_tokens: int = 0
    decode_ms: float = 0.0
    graph_captures: int = 0       # decode steps that had to record a new CUDA graph (filled in by the caller)

    @property
    def prefill_tokens_per_s(self) -> float:
        return self.prefill_tokens / (self.prefill_ms / 1e3) if self.prefill_ms > 0 else 0.0

    @property
    def decode_tokens_per_s(self) -> float:
        return self.decode_tokens / (self.decode_ms / 1e3) if self.decode_ms > 0 else 0.0


def tokens_held(prompt_len: int, max_new_tokens: int, page_size: int) -> int:
    """Cache tokens a request holds at most, rounded up to whole pages.  The
    last generated token is never fed back, so it needs no room."""
    n = prompt_len + max(0, max_new_tokens - 1)
    return (n + page_size - 1) // page_size * page_size


def plan_batch(pending: Sequence[int], prompt_lens: Sequence[int], max_new_tokens: int, batch_size: int,
               capacity_tokens: int, free_slots: int, page_size: int) -> List[int]:
    """The next batch: requests in order, as many as the batch size, the free
    slots and the cache's capacity allow.  At least one, or an error that names
    the request that can never fit."""
    chosen: List[int] = []
    used = 0
    for r in pending:
        if len(chosen) >= min(batch_size, free_slots):
            break
        need = tokens_held(prompt_lens[r], max_new_tokens, page_size)
        if used + need > capacity_tokens:
            break
        chosen.append(r)
        used += need
    if not chosen and pending:
        r = pending[0]
        raise ValueError(
            f"request {r} needs room for {tokens_held(prompt_lens[r], max_new_tokens, page_size)} tokens "
            f"but the cache holds {capacity_tokens} (free slots: {free_slots})")
    return chosen


def plan_prompt_steps(prompt_lens: Sequence[int], max_step_tokens: Optional[int]) -> List[List[Tuple[int, int, int]]]:
    """How a batch's prompts are cut into steps of at most `max_step_tokens` tokens (None or 0: one step
    whatever the size): a list of steps, each a list of (prompt index, first token, end) pieces.  Prompts are
    taken in order and a step is filled before the next begins, so a step holds the end of one prompt, whole
    prompts and the beginning of another; each prompt's pieces follow one another in consecutive steps.  What
    a step's activations need is then bounded by the limit, not by the batch."""
    if not max_step_tokens or sum(prompt_lens) <= max_step_tokens:
        return [[(i, 0, n) for i, n in enumerate(prompt_lens)]]
    steps: List[List[Tuple[int, int, int]]] = [[]]
    room = max_step_tokens
    for i, n in enumerate(prompt_lens):
        start = 0
        while start < n:
            if room == 0:
                steps.append([])
                room = max_step_tokens
            end = min(n, start + room)
            steps[-1].append((i, start, end))
            room -= end - start
            start = end
    return steps


def run_generation(backend: GenerationBackend, prompts: Sequence[Sequence[int]], max_new_tokens: int,
                   stop_token_ids: Sequence[int], batch_size: int, capacity_tokens: int, max_seq_len: int,
                   free_slots: int, page_size: int,
                   callback: Optional[Callable[[int, int], bool]] = None
                   ) -> Tuple[List[List[int]], List[str], GenerationStats]:
    """Returns (generated tokens per request, finish reason per request, stats).
    `callback(request, token)` is called for every accepted token; returning
    False ends that request (reason "stop")."""
    n = len(prompts)
    for i, p in enumerate(prompts):
        if len(p) == 0:
            raise ValueError(f"prompt {i} is empty")
        if len(p) > max_seq_len:
            raise ValueError(f"prompt {i} has {len(p)} tokens, the longest sequence allowed is {max_seq_len}")
    stop = set(int(t) for t in stop_token_ids)
    outputs: List[List[int]] = [[] for _ in range(n)]
    reasons: List[str] = ["length"] * n
    stats = GenerationStats(requests=n)
    if max_new_tokens <= 0:
        return outputs, reasons, stats
    pending = list(range(n))
    prompt_lens = [len(p) for p in prompts]

    def accept(r: int, token: int) -> bool:
        """Record a sampled token; True if the request goes on."""
        if token in stop:
            reasons[r] = "stop"
            return False
        outputs[r].append(token)
        if callback is not None and callback(r, token) is False:
            reasons[r] = "stop"
            return False
        if len(outputs[r]) >= max_new_tokens:
            reasons[r] = "length"
            return False
        if prompt_lens[r] + len(outputs[r]) > max_seq_len:
            # feeding this token would pass the longest length (generation.rs:208-212)
            reasons[r] = "length"
            return False
        return True

    while pending:
        batch = plan_batch(pending, prompt_lens, max_new_tokens, batch_size, capacity_tokens, free_slots,
                           page_size)
        pending = pending[len(batch):]
        stats.batches += 1
        slots: dict = {}
        try:
            for r in batch:
                slots[r] = backend.alloc_slot()
            _run_batch(backend, batch, slots, prompts, prompt_lens, outputs, max_new_tokens, max_seq_len, accept,
                       stats)
        finally:
            # whatever ended the batch (a full cache, a kernel error, a callback that raised, an
            # interrupt): wait for what is still in flight, then every slot it still holds comes back
            if slots:
                try:
                    backend.synchronize()
                finally:
                    for r in list(slots):
                        backend.free_slot(slots.pop(r))
    return outputs, reasons, stats


def _run_batch(backend, batch: Sequence[int], slots: dict, prompts, prompt_lens: Sequence[int],
               outputs: List[List[int]], max_new_tokens: int, max_seq_len: int,
               accept: Callable[[int, int], bool], stats: GenerationStats) -> None:
    """One batch from its prompts to its last token.  `slots` maps request to slot; a request
    that ends gives its slot back at once and leaves the map."""
    backend.synchronize()
    t0 = time.perf_counter()
    first = backend.prefill([slots[r] for r in batch], [prompts[r] for r in batch], batch)
    backend.synchronize()
    stats.prefill_ms += (time.perf_counter() - t0) * 1e3
    stats.prefill_tokens += sum(prompt_lens[r] for r in batch)
    live: List[int] = []
    for r, tok in zip(batch, first):
        if accept(r, int(tok)):
            live.append(r)
        else:
            backend.free_slot(slots.pop(r))
    t0 = time.perf_counter()
    if getattr(backend, "decode_launch", None) is not None:
        _decode_run_ahead(backend, live, slots, outputs, prompt_lens, max_new_tokens, max_seq_len, accept, stats)
    else:
        while live:
            toks = backend.decode([slots[r] for r in live], [outputs[r][-1] for r in live], live,
                                  [len(outputs[r]) for r in live])
            stats.decode_steps += 1
            stats.decode_tokens += len(live)
            still: List[int] = []
            for r, tok in zip(live, toks):
                if accept(r, int(tok)):
                    still.append(r)
                else:
                    backend.free_slot(slots.pop(r))
            live = still
    backend.synchronize()
    stats.decode_ms += (time.perf_counter() - t0) * 1e3


FROM_DEVICE = -1   # as a token handed to `decode_launch`: the token the step before produced for that slot


def _decode_run_ahead(backend, live: List[int], slots: dict, outputs: List[List[int]], prompt_lens: Sequence[int],
                      max_new_tokens: int, max_seq_len: int, accept: Callable[[int, int], bool],
                      stats: GenerationStats) -> None:
    """The decode loop for a backend that can launch a step before the host has
    read the one before (`decode_launch` / `decode_collect`): while the device
    runs step k, step k+1 is laid out and launched for every sequence that
    cannot end by length at step k; its input tokens stay on the device.  A
    sequence that turns out to have met a stop token at step k has one row of
    step k+1 computed in vain; that row is ignored.  The tokens and finish
    reasons are those of the plain loop."""
    def ends_by_length(r: int, produced: int) -> bool:
        # mirrors `accept`: after `produced` tokens the request is over whatever the token is
        return produced >= max_new_tokens or prompt_lens[r] + produced > max_seq_len

    rows = list(live)
    if not rows:
        return
    handle = backend.decode_launch([slots[r] for r in rows], [outputs[r][-1] for r in rows], rows,
                                   [len(outputs[r]) for r in rows])
    dead: set = set()
    while rows:
        # the step after this one: everybody whose next token cannot be the last by length
        ahead = [r for r in rows if r not in dead and not ends_by_length(r, len(outputs[r]) + 1)]
        ahead_handle = None
        if ahead:
            ahead_handle = backend.decode_launch([slots[r] for r in ahead], [FROM_DEVICE] * len(ahead), ahead,
                                                 [len(outputs[r]) + 1 for r in ahead])
        toks = backend.decode_collect(handle)
        stats.decode_steps += 1
        for r, tok in zip(rows, toks):
            if r in dead:
                continue
            stats.decode_tokens += 1
            if not accept(r, int(tok)):
                dead.add(r)
                backend.free_slot(slots.pop(r))
        rows, handle = ahead, ahead_handle
        if rows and all(r in dead for r in rows):
            backend.decode_collect(handle)      # nothing of it is wanted; wait for it all the same
            return
