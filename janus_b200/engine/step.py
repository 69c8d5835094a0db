"""The step function: run the tokens a batch of sequences brings, from the
cache that earlier steps left, and return the logits at the wanted places.

A step's sequences either all bring their prompts (unequal lengths, packed
without padding) or all bring one token; both go through the same code with
per-token positions, so the logits at a position do not depend on how the
tokens were cut into steps or on what else is in the batch.  (The reference runs
one token per row per call with one shared position,
crates/janus-engine/src/model/transformer/forward.rs:25,139-141.)
"""
from __future__ import annotations

import gc
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import log
from ..cache import PAGE_SIZE, CacheFull, CacheView, GroupStepView, SequenceCache
from ..kernels import ops
from .model import DecoderModel
from .workspace import Workspace


FROM_DEVICE = -1   # as a decode step's token: "the token the step before sampled for this slot"
MAX_DECODE_GRAPHS = 48   # captured decode steps kept per engine (one per batch size, page capacity and sampler)


class StepError(ValueError):
    """A step that cannot run: a dead slot, a token outside the vocabulary, a
    sequence past its longest length.  Raised before anything is launched."""


@dataclass
class EngineOptions:
    max_tokens: int = 4096            # tokens the live sequences hold at most (each rounded up to a page)
    max_seq_len: Optional[int] = None  # longest sequence; default: the model's max positions
    max_slots: Optional[int] = None    # live sequences at most; default: one per page, at most 1024
    use_graphs: bool = True            # replay decode steps from CUDA graphs
    # the generation loop cuts a batch's prompts into steps of at most this many tokens (None: one step whatever
    # the size); a step's activations are sized by its tokens, so this bounds them.  The step function itself
    # takes what it is given.
    max_step_tokens: Optional[int] = 32768


@dataclass
class StepEntry:
    slot: int
    tokens: Sequence[int]              # a list, tuple or array of ids (the engine keeps several as an int64 array)
    want: Sequence[int] = ()           # places among `tokens` whose logits are wanted


class StepContext:
    """What a step hands the parts (all tensors int32 on the device)."""

    def __init__(self):
        self.n_tokens = 0
        self.n_seqs = 0
        self.is_decode = False
        self.max_q_len = 0
        self.max_kv_len_bound = 0        # host upper bound of the longest sequence after this step
        self.token_ids: torch.Tensor = None
        self.positions: torch.Tensor = None
        self.token_seq: torch.Tensor = None   # index of each token's sequence within the step
        self.q_start: torch.Tensor = None     # [n_seqs + 1] offsets of each sequence's tokens
        self.kv_len: torch.Tensor = None      # [n_seqs] length of each sequence after this step
        self.seq_slot: torch.Tensor = None    # [n_seqs] cache slot of each sequence
        self.feedback: torch.Tensor = None    # decode only: per slot the token sampled last (for ids < 0)
        self.groups: List[GroupStepView] = []
        self.workspace: Workspace = None
        self.cache: SequenceCache = None
        self.dtype: torch.dtype = None

    def cache_view(self, place: int) -> CacheView:
        cache = self.cache
        gi = cache.group_of_place.get(place)
        if gi is not None:
            g = cache.groups[gi]
            return CacheView(k=g.k[place], v=g.v[place], group=self.groups[gi])
        if place in cache.states:
            return CacheView(state=cache.states[place])
        return CacheView()


def _pad4(n: int) -> int:
    return (n + 3) & ~3


class Engine:
    def __init__(self, model: DecoderModel, options: Optional[EngineOptions] = None):
        self.model = model
        self.options = options or EngineOptions()
        self.device, self.dtype = model.device, model.dtype
        if self.device.type != "cuda":
            raise RuntimeError("the engine runs on a CUDA device only; there is no CPU path")
        o = self.options
        self.max_seq_len = min(o.max_seq_len or model.spec.max_positions, model.spec.max_positions)
        n_pages = max(1, (o.max_tokens + PAGE_SIZE - 1) // PAGE_SIZE)
        n_slots = o.max_slots or min(n_pages, 1024)
        model.limit_positions(self.max_seq_len)
        self.cache = SequenceCache(model.place_cache_specs(), o.max_tokens, n_slots, self.dtype, self.device)
        self.workspace = Workspace(self.device)
        self._pinned: Optional[torch.Tensor] = None
        self._graphs: Dict[Tuple, object] = {}
        self._capture_stream: Optional[torch.cuda.Stream] = None
        self._checked_shapes = set()       # shapes of steps that have run with the kernel faces' checks on
        self.graph_captures = 0            # decode steps that found no captured graph and recorded one
        # logits and sampled tokens of graph steps: one buffer for all graphs (a graph records a view)
        self._graph_logits: Optional[torch.Tensor] = None
        self._graph_tokens = torch.zeros(n_slots, dtype=torch.int32, device=self.device)
        self.last_graph_launches = 0       # kernels of this library in the last step
        self.last_step_h2d_bytes = 0       # bytes of the last step's index buffer
        # per slot: the token sampled last by a graph step, so that the next step can
        # read its input on the device before the host has seen it
        self.feedback = torch.zeros(n_slots, dtype=torch.int32, device=self.device)

    # -- slots -----------------------------------------------------------------
    def alloc_slot(self) -> int:
        return self.cache.alloc_slot()

    def free_slot(self, slot: int) -> None:
        self.cache.free_slot(slot)

    # -- the step --------------------------------------------------------------
    def _validate(self, entries: Sequence[StepEntry], device_tokens: bool = False) -> None:
        if not entries:
            raise StepError("a step needs at least one sequence")
        seen = set()
        V = self.model.vocab_size
        for e in entries:
            if not self.cache.is_live(e.slot):
                raise StepError(f"slot {e.slot} is not held by a live sequence")
            if e.slot in seen:
                raise StepError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"slot {e.slot} brings no tokens")
            if n == 1:
                t = int(e.tokens[0])
                if not (0 <= t < V or (device_tokens and t == FROM_DEVICE)):
                    raise StepError(f"token id {t} is outside the vocabulary of {V}")
            else:
                # one pass over an array, not a Python loop per token (a batch's prompts are tens of
                # thousands); the array stays with the entry for the step's index buffer
                toks = e.tokens = np.asarray(e.tokens, dtype=np.int64).reshape(-1)
                outside = (toks < 0) | (toks >= V)
                if device_tokens:
                    outside &= toks != FROM_DEVICE
                if outside.any():
                    raise StepError(f"token id {int(toks[outside][0])} is outside the vocabulary of {V}")
            if self.cache.lengths[e.slot] + n > self.max_seq_len:
                raise StepError(
                    f"slot {e.slot} would reach {self.cache.lengths[e.slot] + n} tokens, the longest "
                    f"sequence allowed is {self.max_seq_len}")
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise StepError(f"wanted place {w} is outside the {n} tokens that slot {e.slot} brings")

    def _reserve(self, entries: Sequence[StepEntry]) -> None:
        done = []
        try:
            for e in entries:
                self.cache.reserve(e.slot, len(e.tokens))
                done.append(e)
        except CacheFull:
            for e in done:
                for g in self.cache.groups:
                    need = (self.cache.lengths[e.slot] + PAGE_SIZE - 1) // PAGE_SIZE
                    while len(g.pages[e.slot]) > need:
                        g.pool.give_back(g.pages[e.slot].pop())
            raise

    def build_context(self, entries: Sequence[StepEntry], pages_capacity: Optional[int] = None,
                      into: Optional[torch.Tensor] = None):
        """Pack the step's index arrays into one int32 buffer, copy it to the
        device once, and hand out views.  Returns (ctx, want_rows)."""
        cache = self.cache
        S = len(entries)
        lens = [len(e.tokens) for e in entries]
        starts = [cache.lengths[e.slot] for e in entries]
        T = sum(lens)
        after = [s + n for s, n in zip(starts, lens)]
        P = max((a + PAGE_SIZE - 1) // PAGE_SIZE for a in after)
        if pages_capacity is not None:
            if P > pages_capacity:
                raise StepError("a sequence outgrew the page capacity this step was laid out for")
            P = pages_capacity
        wants: List[int] = []
        q_start = [0]
        for e, n in zip(entries, lens):
            wants.extend(q_start[-1] + int(w) for w in e.want)
            q_start.append(q_start[-1] + n)
        W = len(wants)
        G = len(cache.groups)
        sizes = [T, T, T, S + 1, S, S, W] + [T, S * P] * G
        offsets = [0]
        for s in sizes:
            offsets.append(offsets[-1] + _pad4(s))
        host = np.zeros(offsets[-1], dtype=np.int32)
        o = offsets
        host[o[0]:o[0] + T] = np.concatenate([np.asarray(e.tokens, dtype=np.int32) for e in entries])
        host[o[1]:o[1] + T] = np.concatenate([np.arange(s, s + n, dtype=np.int32) for s, n in zip(starts, lens)])
        host[o[2]:o[2] + T] = np.repeat(np.arange(S, dtype=np.int32), lens)
        host[o[3]:o[3] + S + 1] = q_start
        host[o[4]:o[4] + S] = after
        host[o[5]:o[5] + S] = [e.slot for e in entries]
        host[o[6]:o[6] + W] = wants
        for gi, g in enumerate(cache.groups):
            base = 7 + 2 * gi
            host[o[base]:o[base] + T] = np.concatenate(
                [g.dest_rows(e.slot, s, n) for e, s, n in zip(entries, starts, lens)])
            bt = np.full((S, P), -1, dtype=np.int32)
            for i, e in enumerate(entries):
                pages = g.pages[e.slot]
                bt[i, :len(pages)] = pages
            host[o[base + 1]:o[base + 1] + S * P] = bt.reshape(-1)
        total = offsets[-1]
        self.last_step_h2d_bytes = 4 * total
        if self._pinned is None or self._pinned.numel() < total:
            self._pinned = torch.empty(max(total, 4096), dtype=torch.int32, pin_memory=True)
        self._pinned[:total].numpy()[:] = host
        if into is None:
            dev = self._pinned[:total].to(self.device, non_blocking=True)
        else:
            if into.numel() < total:
                raise StepError("the step's index buffer is smaller than this step needs")
            into[:total].copy_(self._pinned[:total], non_blocking=True)
            dev = into
        # The pinned buffer is reused by the next step: wait until this copy has left it.
        copied = torch.cuda.Event()
        copied.record()
        self._copy_done = copied

        def seg(i: int, n: int) -> torch.Tensor:
            return dev[offsets[i]:offsets[i] + n]

        ctx = StepContext()
        ctx.n_tokens, ctx.n_seqs = T, S
        ctx.is_decode = all(n == 1 for n in lens)
        ctx.max_q_len = max(lens)
        ctx.max_kv_len_bound = P * PAGE_SIZE
        ctx.token_ids, ctx.positions, ctx.token_seq = seg(0, T), seg(1, T), seg(2, T)
        ctx.q_start, ctx.kv_len, ctx.seq_slot = seg(3, S + 1), seg(4, S), seg(5, S)
        ctx.groups = [GroupStepView(seg(7 + 2 * gi, T), seg(8 + 2 * gi, S * P).view(S, P), PAGE_SIZE)
                      for gi in range(G)]
        ctx.workspace, ctx.cache, ctx.dtype = self.workspace, cache, self.dtype
        return ctx, seg(6, W), total

    def step(self, entries: Sequence[StepEntry], borrow: bool = False) -> torch.Tensor:
        """Run one step; returns float32 logits [number of wanted places, vocab]
        on the device, in the order of the entries and of their `want`.

        With `borrow` the result may be a buffer that the next step overwrites
        (the generation loop samples from it at once); otherwise it is the
        caller's own."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        self._validate(entries)
        self._reserve(entries)
        if log.enabled("debug"):
            log.log("debug", f"step: {len(entries)} sequences, {sum(len(e.tokens) for e in entries)} tokens, "
                             f"{sum(len(e.want) for e in entries)} wanted rows")
        if (self.options.use_graphs and all(len(e.tokens) == 1 and tuple(e.want) == (0,) for e in entries)):
            with log.nvtx_range("decode step (graph)"):
                logits = self._graph_decode(entries, None)[0]
            if not borrow:
                logits = logits.clone()
        else:
            if getattr(self, "_copy_done", None) is not None:
                self._copy_done.synchronize()
            ctx, want_rows, _ = self.build_context(entries)
            logits = torch.empty((want_rows.shape[0], self.model.vocab_size), dtype=torch.float32,
                                 device=self.device)
            before = ops.launch_count()
            # a step of a shape that has run before hands the same kinds of tensors to the same kernels:
            # the faces' checks of device, dtype and shape are made the first time only
            shape = (ctx.n_tokens, ctx.n_seqs, ctx.max_q_len, ctx.max_kv_len_bound, want_rows.shape[0])
            if shape in self._checked_shapes:
                with ops.unchecked(), log.nvtx_range(f"step of {ctx.n_tokens} tokens"):
                    self.model.forward(ctx, want_rows, logits)
            else:
                with log.nvtx_range(f"step of {ctx.n_tokens} tokens (first of its shape)"):
                    self.model.forward(ctx, want_rows, logits)
                if len(self._checked_shapes) >= 4096:
                    self._checked_shapes.clear()
                self._checked_shapes.add(shape)
            self.last_graph_launches = ops.launch_count() - before
        for e in entries:
            self.cache.advance(e.slot, len(e.tokens))
        return logits

    def profile_step(self, entries: Sequence[StepEntry]) -> dict:
        """Run one step with its kernels launched one by one and timed by CUDA events: which kernels the step
        launches, how often, and how long the stream spends on each.  The step counts (the cache takes its
        tokens).  Returns {"tokens", "sequences", "kind", "total_ms", "kernels": [{"name", "launches", "ms"}]}
        with the kernels in the order of their first launch."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        graphs, self.options.use_graphs = self.options.use_graphs, False
        try:
            torch.cuda.synchronize(self.device)
            with ops.trace_launches() as events:
                self.step(entries)
            torch.cuda.synchronize(self.device)
        finally:
            self.options.use_graphs = graphs
        rows: Dict[str, list] = {}
        for (_, _, before), (name, kernels, after) in zip(events, events[1:]):
            row = rows.setdefault(name, [0, 0.0])
            row[0] += kernels
            row[1] += before.elapsed_time(after)
        lens = [len(e.tokens) for e in entries]
        return {"tokens": sum(lens), "sequences": len(entries),
                "kind": "decode" if all(n == 1 for n in lens) else "prompt",
                "total_ms": round(events[0][2].elapsed_time(events[-1][2]), 4) if len(events) > 1 else 0.0,
                "kernels": [{"name": k, "launches": v[0], "ms": round(v[1], 4)} for k, v in rows.items()]}

    def decode_sample(self, slots: Sequence[int], tokens: Sequence[int], sampler, requests: Sequence[int],
                      steps: Sequence[int]) -> torch.Tensor:
        """One token per sequence in, the sampled next token of each out (int32
        on the device, a buffer that the next call overwrites).  Forward pass and
        sampling replay from one CUDA graph; `requests` and `steps` key the
        sampler's random numbers.  A token FROM_DEVICE stands for the token that
        the call before sampled for that slot, so that a step can be launched
        before the host has read the last one's result."""
        entries = [StepEntry(s, (int(t),), (0,)) for s, t in zip(slots, tokens)]
        self._validate(entries, device_tokens=self.options.use_graphs)
        self._reserve(entries)
        if self.options.use_graphs:
            out = self._graph_decode(entries, (sampler, requests, steps))[1]
        else:
            if getattr(self, "_copy_done", None) is not None:
                self._copy_done.synchronize()
            ctx, want_rows, _ = self.build_context(entries)
            logits = torch.empty((len(entries), self.model.vocab_size), dtype=torch.float32, device=self.device)
            self.model.forward(ctx, want_rows, logits)
            meta = torch.tensor([list(requests), list(steps), list(slots)], dtype=torch.int32).to(self.device)
            out = sampler.sample(logits, meta[0], meta[1], meta[2])
        for e in entries:
            self.cache.advance(e.slot, 1)
        return out

    # -- decode steps replayed from CUDA graphs -----------------------------------
    def _graph_decode(self, entries: Sequence[StepEntry], sampling):
        """One token per sequence, every sequence's logits wanted: the kernels of
        the step (and of sampling, if asked for) are captured once per (batch
        size, page capacity, sampler) and replayed; a replay only refreshes the
        step's index buffer.  The capacity is the pages of the longest sequence,
        rounded up to a power of two, so that a graph serves many steps before a
        sequence outgrows it.  Returns (logits, sampled tokens or None)."""
        B = len(entries)
        need = max((self.cache.lengths[e.slot] + 1 + PAGE_SIZE - 1) // PAGE_SIZE for e in entries)
        cap = 1
        while cap < need:
            cap *= 2
        sampler = sampling[0] if sampling is not None else None
        # a graph bakes in the sampler's options, seed and count table: samplers equal in those share it
        key = (B, cap, self.workspace.generation, sampler.graph_key() if sampler is not None else 0)
        rec = self._graphs.get(key)
        if rec is None:
            for k in [k for k in self._graphs if k[2] != self.workspace.generation]:
                del self._graphs[k]          # buffers moved: those graphs hold stale addresses
            rec = _DecodeGraph(self, B, cap, sampler)
            rec.fill(entries, sampling)
            rec.run_forward()                # direct: this run is the step
            torch.cuda.synchronize(self.device)
            key = (B, cap, self.workspace.generation, key[3])
            graph = torch.cuda.CUDAGraph()
            before = ops.launch_count()
            # No garbage collection while capturing: collecting an older engine would destroy
            # its CUDA graphs in the middle of this capture, which invalidates it.  The capture is
            # begun and ended by hand on a stream of its own: `torch.cuda.graph` would synchronise,
            # run a full collection (25 ms) and empty the allocator's cache at every new graph.
            gc_was_on = gc.isenabled()
            gc.disable()
            try:
                if self._capture_stream is None:
                    self._capture_stream = torch.cuda.Stream(device=self.device)
                side = self._capture_stream
                side.wait_stream(torch.cuda.current_stream(self.device))
                with torch.cuda.stream(side), ops.unchecked():      # the direct run above made the checks
                    graph.capture_begin()
                    try:
                        rec.run_forward()
                    finally:
                        graph.capture_end()
                torch.cuda.current_stream(self.device).wait_stream(side)
            finally:
                if gc_was_on:
                    gc.enable()
            rec.graph, rec.launches = graph, ops.launch_count() - before
            self.graph_captures += 1
            while len(self._graphs) >= MAX_DECODE_GRAPHS:      # keep the ones used last
                del self._graphs[next(iter(self._graphs))]
            self._graphs[key] = rec
        else:
            self._graphs[key] = self._graphs.pop(key)          # used last: to the end of the line
            rec.fill(entries, sampling)
            rec.graph.replay()
        self.last_graph_launches = rec.launches
        self.last_step_h2d_bytes = 4 * rec.total
        return rec.logits, rec.tokens_out

    def _graph_output_buffers(self, B: int):
        """Views for B rows of the logits and token buffers that all captured steps share.  A batch
        larger than any before gets a larger buffer; graphs recorded on the old one keep it alive."""
        V = self.model.vocab_size
        if self._graph_logits is None or self._graph_logits.shape[0] < B:
            rows = 8
            while rows < B:
                rows *= 2
            rows = min(rows, max(self.cache.n_slots, B))
            self._graph_logits = torch.empty((rows, V), dtype=torch.float32, device=self.device)
        return self._graph_logits[:B], self._graph_tokens[:B]


class _DecodeGraph:
    """The fixed buffers of one captured decode step and the fast refill of its
    index buffer: two pinned host copies alternate so that a refill never
    overwrites a copy still in flight."""

    def __init__(self, engine: "Engine", B: int, cap: int, sampler):
        self.engine, self.B, self.cap, self.sampler = engine, B, cap, sampler
        cache = engine.cache
        G = len(cache.groups)
        sizes = [B, B, B, B + 1, B, B, B] + [B, B * cap] * G + [B, B, B]
        self.offsets = [0]
        for n in sizes:
            self.offsets.append(self.offsets[-1] + _pad4(n))
        self.total = self.offsets[-1]
        self.extra = 7 + 2 * G                      # first of the three sampling segments
        dev = engine.device
        self.meta = torch.zeros(self.total, dtype=torch.int32, device=dev)
        self.logits, tokens_out = engine._graph_output_buffers(B)
        self.tokens_out = tokens_out if sampler is not None else None
        self.host = [torch.zeros(self.total, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self.host_np = [h.numpy() for h in self.host]
        o = self.offsets
        for h in self.host_np:                      # the parts that never change
            h[o[2]:o[2] + B] = np.arange(B)
            h[o[3]:o[3] + B + 1] = np.arange(B + 1)
            h[o[6]:o[6] + B] = np.arange(B)
            for gi in range(G):
                h[o[8 + 2 * gi]:o[8 + 2 * gi] + B * cap] = -1
        self.row_sig = [[[None] * B for _ in range(G)] for _ in range(2)]
        self.events = [None, None]
        self.flip = 0
        self.graph, self.launches = None, 0

        def seg(i: int, n: int) -> torch.Tensor:
            return self.meta[o[i]:o[i] + n]

        ctx = StepContext()
        ctx.n_tokens, ctx.n_seqs, ctx.is_decode, ctx.max_q_len = B, B, True, 1
        ctx.max_kv_len_bound = cap * PAGE_SIZE
        ctx.token_ids, ctx.positions, ctx.token_seq = seg(0, B), seg(1, B), seg(2, B)
        ctx.q_start, ctx.kv_len, ctx.seq_slot = seg(3, B + 1), seg(4, B), seg(5, B)
        ctx.groups = [GroupStepView(seg(7 + 2 * gi, B), seg(8 + 2 * gi, B * cap).view(B, cap), PAGE_SIZE)
                      for gi in range(G)]
        ctx.workspace, ctx.cache, ctx.dtype = engine.workspace, cache, engine.dtype
        ctx.feedback = engine.feedback
        self.ctx, self.want_rows = ctx, seg(6, B)
        self.sample_meta = (seg(self.extra, B), seg(self.extra + 1, B), seg(self.extra + 2, B))

    def run_forward(self) -> None:
        self.engine.model.forward(self.ctx, self.want_rows, self.logits)
        if self.sampler is not None:
            requests, steps, count_rows = self.sample_meta
            self.sampler.sample_into(self.logits, self.tokens_out, requests, steps, count_rows,
                                     self.engine.feedback)

    def fill(self, entries: Sequence[StepEntry], sampling) -> None:
        B, cap, o = self.B, self.cap, self.offsets
        cache = self.engine.cache
        k = self.flip
        self.flip ^= 1
        if self.events[k] is not None:
            self.events[k].synchronize()
        h = self.host_np[k]
        slots = [e.slot for e in entries]
        lens = [cache.lengths[s] for s in slots]
        h[o[0]:o[0] + B] = [e.tokens[0] for e in entries]
        h[o[1]:o[1] + B] = lens
        h[o[4]:o[4] + B] = [n + 1 for n in lens]
        h[o[5]:o[5] + B] = slots
        for gi, g in enumerate(cache.groups):
            pages = g.pages
            h[o[7 + 2 * gi]:o[7 + 2 * gi] + B] = [pages[s][n // PAGE_SIZE] * PAGE_SIZE + n % PAGE_SIZE
                                                  for s, n in zip(slots, lens)]
            table = h[o[8 + 2 * gi]:o[8 + 2 * gi] + B * cap].reshape(B, cap)
            sigs = self.row_sig[k][gi]
            windowed = g.spec.window > 0
            for i, s in enumerate(slots):
                row = pages[s]
                sig = (s, cache.epochs[s], len(row))
                if windowed or sigs[i] != sig:       # a window group's rows lose pages as they pass
                    table[i, :len(row)] = row
                    table[i, len(row):] = -1
                    sigs[i] = sig
        if sampling is not None:
            _, requests, steps = sampling
            e0 = self.extra
            h[o[e0]:o[e0] + B] = requests
            h[o[e0 + 1]:o[e0 + 1] + B] = steps
            h[o[e0 + 2]:o[e0 + 2] + B] = slots
        self.meta.copy_(self.host[k], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.events[k] = ev
