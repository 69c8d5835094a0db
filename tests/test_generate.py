"""Generation through the Python entry point, compared with the plain
implementation: greedy tokens, long decoding, the first tokens of a sequence,
stop tokens and early finish in a batch, temperature sampling that does not
depend on the batch, and errors raised before anything is launched."""
import pytest
import torch

import plain_llama as P
from helpers import BF16_TOL, TINY, make_model_dir, random_tokens, rel_err, tol_for

pytestmark = pytest.mark.gpu


def load(tmp_path, name, dtype, seed=3, **kw):
    import janus_b200
    d = make_model_dir(TINY[name], str(tmp_path / f"m{name}{dtype}"), seed=seed, dtype=dtype)
    kw.setdefault("max_tokens", 2048)
    return janus_b200.load(d, dtype=dtype, **kw), P.read_model_dir(d)


def check_greedy_against_plain(cfg, w, prompt, produced, dtype):
    """Teacher-forced: every produced token is the plain argmax given the tokens
    before it; in bfloat16 a token whose plain logit lies within the tolerance of
    the maximum is accepted as well."""
    logits = P.forward(cfg, w, list(prompt) + list(produced))
    for j, tok in enumerate(produced):
        row = logits[len(prompt) - 1 + j]
        if dtype == "float32":
            assert tok == P.argmax_lowest(row), f"token {j}"
        else:
            assert float(row.max() - row[tok]) <= BF16_TOL * float(row.abs().max()), f"token {j}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_of_unequal_prompts(tmp_path, name, dtype):
    model, (cfg, w) = load(tmp_path, name, dtype)
    lens = {"A": [5, 11, 17], "B": [1, 7, 33, 64]}[name]
    prompts = [random_tokens(n, cfg["vocab_size"], 7 + n) for n in lens]
    out, reasons, stats = model.generate(prompts, max_tokens=8, ignore_eos=True, return_reasons=True)
    assert [len(o) for o in out] == [8] * len(prompts) and reasons == ["length"] * len(prompts)
    assert stats.prefill_tokens == sum(lens) and stats.decode_steps == 7
    for p, o in zip(prompts, out):
        check_greedy_against_plain(cfg, w, p, o, dtype)
        if dtype == "float32":
            assert o == P.generate(cfg, w, p, 8)
    # the same requests in batches of two, one batch after another, give the same tokens
    out2, _ = model.generate(prompts, max_tokens=8, ignore_eos=True, batch_size=2)
    assert out2 == out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("limit", [1, 7, 40])
def test_prompts_cut_into_steps_of_limited_size_give_the_same_tokens(tmp_path, dtype, limit):
    """`max_step_tokens`: the batch's prompts run in steps of at most that many tokens (a step holds the end of
    one prompt, whole prompts and the beginning of another; with a limit of 1 every token is a step of its
    own).  The first sampled tokens come from different steps' logits; everything matches the plain
    implementation as the uncut prompts do."""
    model, (cfg, w) = load(tmp_path, "B", dtype, max_step_tokens=limit)
    lens = [1, 7, 33, 64, 2]
    prompts = [random_tokens(n, cfg["vocab_size"], 11 + n) for n in lens]
    out, stats = model.generate(prompts, max_tokens=6, ignore_eos=True)
    assert stats.prefill_tokens == sum(lens)
    for p, o in zip(prompts, out):
        check_greedy_against_plain(cfg, w, p, o, dtype)
        if dtype == "float32":
            assert o == P.generate(cfg, w, p, 6)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(tmp_path, dtype):
    model, (cfg, w) = load(tmp_path, "A", dtype)
    prompt = random_tokens(3, 256, 1)
    out, _ = model.generate([prompt], max_tokens=125, ignore_eos=True)       # up to the 128 positions of the model
    assert len(out[0]) == 125
    check_greedy_against_plain(cfg, w, prompt, out[0], dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(tmp_path, dtype):
    from janus_b200.engine import StepEntry
    model, (cfg, w) = load(tmp_path, "B", dtype)
    ids = random_tokens(4, 384, 2)
    ref = P.forward(cfg, w, ids)
    s = model.alloc_slot()
    rows = [model.step([StepEntry(s, [t], [0])]).cpu() for t in ids]          # positions 0, 1, 2, 3 one by one
    assert rel_err(torch.cat(rows), ref) < tol_for(dtype)
    model.free_slot(s)


def test_stop_tokens_end_sequences_early(tmp_path):
    model, (cfg, w) = load(tmp_path, "A", "float32")
    prompts = [random_tokens(n, 256, 30 + n) for n in (4, 9, 6)]
    free = P.generate(cfg, w, prompts[1], 12)
    stop = free[4]                                            # request 1 meets its 5th token as a stop token
    want = [P.generate(cfg, w, p, 12, stop_ids=[stop]) for p in prompts]
    out, reasons, stats = model.generate(prompts, max_tokens=12, stop_token_ids=[stop], ignore_eos=True,
                                         return_reasons=True)
    assert out == want and len(out[1]) <= 4 and reasons[1] == "stop"
    assert all(r == ("stop" if len(o) < 12 else "length") for o, r in zip(out, reasons))
    assert model.engine.cache.n_free_slots == model.engine.cache.n_slots     # every slot came back
    model.engine.cache.check()
    # config.json's eos ids stop too unless ignored
    eos = TINY["A"]["eos_token_id"]
    out2, reasons2, _ = model.generate(prompts, max_tokens=12, stop_token_ids=[stop], return_reasons=True)
    assert all(t not in eos for o in out2 for t in o)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_temperature_sampling_is_seeded_and_independent_of_the_batch(tmp_path, dtype):
    model, (cfg, w) = load(tmp_path, "B", dtype)
    prompts = [random_tokens(n, 384, 50 + n) for n in (1, 7, 33, 64)]
    kw = dict(max_tokens=16, temperature=0.8, seed=1234, ignore_eos=True)
    a, _ = model.generate(prompts, **kw)
    b, _ = model.generate(prompts, **kw)
    c, _ = model.generate(prompts, batch_size=1, **kw)
    d, _ = model.generate(prompts, **dict(kw, seed=99))
    assert a == b == c and a != d
    # every sampled token against the plain sampler, step by step along the engine's own sequence: with the
    # step's uniform number u, the token's interval of the cumulative distribution (in index order) must hold u,
    # give or take what the logits' tolerance moves a boundary by
    slack = 2e-4 if dtype == "float32" else 2e-2
    for i, (p, o) in enumerate(zip(prompts, a)):
        assert len(o) == 16
        for j, tok in enumerate(o):
            probs = P.sampling_distribution(P.forward(cfg, w, p + o[:j])[-1], 0.8).double()
            cdf = torch.cumsum(probs, 0)
            u = P.uniform_for(1234, i, j)
            lo = float(cdf[tok - 1]) if tok > 0 else 0.0
            assert lo - slack <= u < float(cdf[tok]) + slack, \
                f"request {i} step {j}: token {tok} holds [{lo:.6f}, {float(cdf[tok]):.6f}), u = {u:.6f}"
    e, _ = model.generate(prompts[:2], max_tokens=6, temperature=0.7, top_k=5, top_p=0.9, repetition_penalty=1.3,
                          seed=3, ignore_eos=True)
    for p, o in zip(prompts[:2], e):
        for j, tok in enumerate(o):
            logits = P.forward(cfg, w, p + o[:j])[-1]
            probs = P.sampling_distribution(logits, 0.7, 5, 0.9, 1.3, o[:j])
            # tokens near the cut-off can fall either way in bfloat16; in float32 the kept set is plain's
            if dtype == "float32":
                assert probs[tok] > 0


def test_command_line(tmp_path):
    """`<model_dir> "<prompt>" --max-tokens N --temperature T`, as the reference's examples take them."""
    import json
    import os
    import subprocess
    import sys
    from helpers import ROOT
    d = make_model_dir(TINY["A"], str(tmp_path / "m"), seed=3, dtype="float32")
    cfg, w = P.read_model_dir(d)
    prompts = [random_tokens(6, 256, 1), random_tokens(3, 256, 2), random_tokens(9, 256, 3)]
    cmd = [sys.executable, os.path.join(ROOT, "bin", "janus_b200"), d] + [",".join(map(str, p)) for p in prompts] + \
          ["--max-tokens", "5", "--batch-size", "2", "--temperature", "0.0", "--dtype", "float32", "--ignore-eos", "--json"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    got = json.loads(res.stdout.strip().splitlines()[-1])
    assert got["tokens"] == [P.generate(cfg, w, p, 5) for p in prompts]
    assert got["finish_reasons"] == ["length"] * 3
    bad = subprocess.run(cmd[:3] + ["1,x,3"], capture_output=True, text=True, timeout=120)
    assert bad.returncode != 0 and "token ids" in (bad.stderr + bad.stdout)
    # what the library refuses is one line and exit code 1, not a traceback: a token outside the vocabulary,
    # a folder that is not there
    for args in ([cmd[2], "1,99999,3"], [str(tmp_path / "nowhere"), "1,2"]):
        refused = subprocess.run(cmd[:2] + args, capture_output=True, text=True, timeout=120)
        assert refused.returncode == 1 and refused.stderr.strip().splitlines()[-1].startswith("Error: ")
        assert "Traceback" not in refused.stderr
    # the longer spellings of the same options, prompts given as options and from a file
    listing = tmp_path / "prompts.txt"
    listing.write_text(" ".join(map(str, prompts[2])) + "\n")
    alias = cmd[:3] + ["--prompt-ids", ",".join(map(str, prompts[0])), "--prompt-ids", ",".join(map(str, prompts[1])),
                       "--prompt-ids-file", str(listing), "--max-new-tokens", "5", "--max-batch", "2", "--dtype", "fp32",
                       "--max-seq-len", "64", "--ignore-eos", "--json"]
    res = subprocess.run(alias, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    assert json.loads(res.stdout.strip().splitlines()[-1])["tokens"] == got["tokens"]
    # a folder with config.json only, run with seeded random weights: the same seed gives the same tokens
    only_config = tmp_path / "c"
    only_config.mkdir()
    (only_config / "config.json").write_text(json.dumps(TINY["A"]))
    rnd = [sys.executable, os.path.join(ROOT, "bin", "janus_b200"), str(only_config), "1,2,3", "--random-weights",
           "--seed-weights", "7", "--max-tokens", "4", "--ignore-eos", "--json"]
    runs = [subprocess.run(rnd, capture_output=True, text=True, timeout=300) for _ in range(2)]
    assert all(r.returncode == 0 for r in runs), runs[0].stderr[-2000:]
    outs = [json.loads(r.stdout.strip().splitlines()[-1])["tokens"] for r in runs]
    assert outs[0] == outs[1] and len(outs[0][0]) == 4


def test_errors_before_launch(tmp_path):
    from janus_b200.cache import CacheFull
    from janus_b200.engine import StepEntry, StepError
    model, _ = load(tmp_path, "A", "float32", max_tokens=128)
    s = model.alloc_slot()
    with pytest.raises(StepError, match="vocabulary"):
        model.step([StepEntry(s, [1, 256], [0])])
    with pytest.raises(StepError, match="longest"):
        model.step([StepEntry(s, [1] * 129, [0])])
    with pytest.raises(StepError, match="not held"):
        model.step([StepEntry(s + 1, [1], [0])])
    with pytest.raises(StepError, match="wanted place"):
        model.step([StepEntry(s, [1, 2], [2])])
    t = model.alloc_slot()
    model.step([StepEntry(s, [1] * 100, [])])
    with pytest.raises(CacheFull):
        model.step([StepEntry(t, [1] * 10, [])])           # both pages are held by the first sequence
    assert model.engine.cache.length(s) == 100 and model.engine.cache.length(t) == 0
    model.engine.cache.check()
    model.free_slot(s)
    assert model.step([StepEntry(t, [1] * 10, [9])]).shape == (1, 256)


def test_profile_lists_the_kernels_of_a_prompt_step_and_of_a_decode_step(tmp_path):
    """`Model.profile` (the command line's --profile): every kernel face of the two steps with its launches and
    its time on the stream; the times add up to the step's; the slots come back; logits are untouched by it."""
    model, (cfg, w) = load(tmp_path, "A", "bfloat16")
    prompts = [random_tokens(n, 256, 80 + n) for n in (70, 9)]
    before, _ = model.generate(prompts, max_tokens=4, ignore_eos=True)
    prof = model.profile(prompts)
    for part, kind, tokens in (("prefill", "prompt", 79), ("decode", "decode", 2)):
        step = prof[part]
        assert step["kind"] == kind and step["tokens"] == tokens and step["sequences"] == 2
        names = [k["name"] for k in step["kernels"]]
        assert names[0] == "embed_gather" and "rmsnorm" in names
        for product in ("qkv", "o", "gate_up", "down", "head"):
            assert any(n.startswith("gemm_bf16") and n.endswith(" " + product) for n in names), (product, names)
        assert any(n.startswith("attention") for n in names)
        layers = cfg["num_hidden_layers"]
        assert next(k for k in step["kernels"] if k["name"] == "rmsnorm")["launches"] == 2 * layers + 1
        assert all(k["ms"] >= 0.0 and k["launches"] >= 1 for k in step["kernels"])
        assert abs(sum(k["ms"] for k in step["kernels"]) - step["total_ms"]) < 1e-2 * max(1.0, step["total_ms"])
    assert model.engine.cache.n_free_slots == model.engine.cache.n_slots
    after, _ = model.generate(prompts, max_tokens=4, ignore_eos=True)
    assert after == before
