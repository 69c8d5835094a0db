"""Trace replay through `bin/trace_run`, compared with the plain implementation:
each request alone and whole; with the last 32 tokens one by one; and in batches
of unequal lengths whose shorter requests end earlier, one batch after another
so that slots and pages are used again.  In float32 and in bfloat16, for both
tiny configurations."""
import numpy as np
import pytest
import torch

import plain_llama as P
from helpers import TINY, TraceRun, make_model_dir, random_tokens, rel_err, tol_for

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 11, 70, 17, 40, 100], "B": [1, 7, 64, 33, 130, 90]}


@pytest.fixture(scope="module")
def plain_logits():
    return {}


@pytest.mark.parametrize("graphs", [True, False], ids=["graphs", "no-graphs"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_replay_matches_plain_however_the_tokens_are_cut(tmp_path, name, dtype, graphs):
    cfg = TINY[name]
    model_dir = make_model_dir(cfg, str(tmp_path / "model"), seed={"A": 0, "B": 1}[name], dtype=dtype)
    pcfg, pw = P.read_model_dir(model_dir)
    reqs = {f"r{i}": random_tokens(n, cfg["vocab_size"], 100 + i) for i, n in enumerate(LENGTHS[name])}
    ref = {rid: P.forward(pcfg, pw, ids).numpy() for rid, ids in reqs.items()}
    tol = tol_for(dtype)
    # room for 5 pages: two batches cannot be live at once, so pages and slots are used again
    run = TraceRun(model_dir, dtype, str(tmp_path / "out"), max_tokens=320, graphs=graphs)
    try:
        # 1. each request alone and whole
        for rid, ids in reqs.items():
            got = run.step([{"id": rid, "tokens": ids, "want": list(range(len(ids)))}], end=[rid])
            assert rel_err(got, ref[rid]) < tol, f"{rid} whole"
        # 2. the last 32 tokens one by one
        for rid, ids in reqs.items():
            cut = max(1, len(ids) - 32)
            rows = [run.step([{"id": "x" + rid, "tokens": ids[:cut], "want": list(range(cut))}])]
            for j in range(cut, len(ids)):
                rows.append(run.step([{"id": "x" + rid, "tokens": [ids[j]], "want": [0]}],
                                     end=["x" + rid] if j == len(ids) - 1 else []))
            if cut == len(ids):
                run.step([], end=["x" + rid])
            got = np.concatenate(rows, axis=0)
            err = rel_err(got, ref[rid])
            first_bad = int(np.argmax(np.abs(got - ref[rid]).max(axis=1) > tol * np.abs(ref[rid]).max()))
            assert err < tol, f"{rid} one by one: first wrong position {first_bad} (prefix {cut})"
        # 3. batches of unequal lengths; shorter requests end earlier; batch after batch
        names = list(reqs)
        for batch in (names[:3], names[3:5], names[5:] + names[:1]):
            prompt = {rid: max(1, len(reqs[rid]) // 2) for rid in batch}
            got = {rid: [] for rid in batch}
            out = run.step([{"id": "b" + rid, "tokens": reqs[rid][:prompt[rid]], "want": list(range(prompt[rid]))}
                            for rid in batch],
                           end=["b" + rid for rid in batch if prompt[rid] == len(reqs[rid])])
            at = 0
            for rid in batch:
                got[rid].append(out[at:at + prompt[rid]])
                at += prompt[rid]
            live = [rid for rid in batch if prompt[rid] < len(reqs[rid])]
            pos = dict(prompt)
            while live:
                ending = [rid for rid in live if pos[rid] == len(reqs[rid]) - 1]
                out = run.step([{"id": "b" + rid, "tokens": [reqs[rid][pos[rid]]], "want": [0]} for rid in live],
                               end=["b" + rid for rid in ending])
                for i, rid in enumerate(live):
                    got[rid].append(out[i:i + 1])
                    pos[rid] += 1
                live = [rid for rid in live if rid not in ending]
            for rid in batch:
                g = np.concatenate(got[rid], axis=0)
                bad = np.abs(g - ref[rid]).max(axis=1) > tol * np.abs(ref[rid]).max()
                assert rel_err(g, ref[rid]) < tol, \
                    f"{rid} in batch {batch}: first wrong position {int(np.argmax(bad))} (prompt {prompt[rid]})"
    finally:
        code = run.close()
    assert code == 0


def test_steps_without_wanted_logits_write_no_file(tmp_path):
    cfg = TINY["A"]
    model_dir = make_model_dir(cfg, str(tmp_path / "model"), seed=0, dtype="float32")
    pcfg, pw = P.read_model_dir(model_dir)
    ids = random_tokens(20, cfg["vocab_size"], 5)
    run = TraceRun(model_dir, "float32", str(tmp_path / "out"), max_tokens=64)
    try:
        assert run.step([{"id": "a", "tokens": ids[:12], "want": []}]).size == 0
        got = run.step([{"id": "a", "tokens": ids[12:], "want": [7]}], end=["a"])
    finally:
        assert run.close() == 0
    assert rel_err(got, P.forward(pcfg, pw, ids).numpy()[19:20]) < tol_for("float32")
