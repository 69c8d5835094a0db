"""Seeded random schedules through the step function: requests come and go, every step picks some of the live
requests and hands each either the next chunk of its tokens (any length) or a single token, chunks and single
tokens mixed in one step; requests that are through give their slot back and new ones take it.  Whatever the
cut, every logit row must match the plain implementation's row for that request and position, in float32
and in bfloat16."""
import random
import tempfile

import numpy as np
import pytest

import plain_llama as P
from helpers import TINY, make_model_dir, random_tokens, tol_for

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name, seed", [("A", 1), ("A", 2), ("B", 3), ("B", 4)])
def test_random_schedules_match_plain(name, seed, dtype):
    import janus_b200
    from janus_b200.engine import StepEntry
    cfg = TINY[name]
    rng = random.Random(1000 * seed + (dtype == "float32"))
    with tempfile.TemporaryDirectory() as d:
        make_model_dir(cfg, d, seed=seed, dtype=dtype)
        c, w = P.read_model_dir(d)
        # room for four live requests of the longest length: a full cache is no subject of this test
        model = janus_b200.load(d, dtype=dtype, max_tokens=4 * cfg["max_position_embeddings"], max_slots=4)
    top = cfg["max_position_embeddings"]
    lengths = [rng.choice([1, 2, 7, 30, 63, 64, 65, 100, top - 1, top]) for _ in range(10)]
    requests = [random_tokens(n, cfg["vocab_size"], 50 * seed + i) for i, n in enumerate(lengths)]
    ref = [P.forward(c, w, ids).numpy() for ids in requests]
    scale = [float(np.abs(r).max()) for r in ref]
    tol = tol_for(dtype)
    waiting = list(range(len(requests)))
    live = {}                                    # request -> [slot, tokens done]
    steps = 0
    while waiting or live:
        while waiting and len(live) < 4 and rng.random() < 0.7:
            live[waiting.pop(0)] = [model.alloc_slot(), 0]
        if not live:
            continue
        chosen = [r for r in live if rng.random() < 0.75] or [next(iter(live))]
        entries, rows = [], []
        for r in chosen:
            slot, done = live[r]
            left = len(requests[r]) - done
            kind = rng.random()
            n = 1 if kind < 0.4 else min(left, rng.choice([1, 2, 5, 17, 40, 64, 90, left]))
            want = sorted(rng.sample(range(n), rng.randint(0, min(n, 6)))) if rng.random() < 0.8 else list(range(n))
            if n == 1 and rng.random() < 0.7:
                want = [0]
            entries.append(StepEntry(slot, requests[r][done:done + n], want))
            rows += [(r, done + j) for j in want]
            live[r][1] = done + n
        out = model.step(entries).cpu().numpy()
        steps += 1
        assert out.shape[0] == len(rows)
        for got, (r, pos) in zip(out, rows):
            err = float(np.abs(got - ref[r][pos]).max()) / scale[r]
            assert err < tol, f"step {steps}: request {r} (length {lengths[r]}) position {pos}: {err:.2e}"
        for r in [r for r in live if live[r][1] == len(requests[r])]:
            model.free_slot(live.pop(r)[0])
    model.check()
    model.engine.cache.check()
    assert model.engine.cache.n_free_slots == 4
