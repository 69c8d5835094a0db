"""One layer with the Llama-3.1-8B sizes (hidden 4096, 32 heads over 8 kv heads of
128, intermediate 14336, llama3 rope scaling) and a small vocabulary, against the
plain implementation, in float32 and in bfloat16: a prompt in one step, the rest
token by token across page boundaries, and two sequences of unequal length in
one batch.  The product path's tile sizes, split-K and key splits are those of
the full model, which the tiny configurations never reach; a prompt of 600
tokens runs the products that work in CTA pairs."""
import numpy as np
import pytest
import torch

import plain_llama as P
from helpers import make_model_dir, random_tokens, rel_err, tol_for

pytestmark = pytest.mark.gpu

BIG_LAYER = dict(
    architectures=["LlamaForCausalLM"], hidden_size=4096, num_hidden_layers=1, num_attention_heads=32,
    num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=2048, max_position_embeddings=1024,
    rms_norm_eps=1e-5, rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=256),
    tie_word_embeddings=False)


@pytest.fixture(scope="module")
def big_model(tmp_path_factory):
    d = make_model_dir(BIG_LAYER, str(tmp_path_factory.mktemp("big") / "m"), seed=11, dtype="bfloat16", sharpen=1.5)
    cfg, w = P.read_model_dir(d)
    ids = [random_tokens(n, BIG_LAYER["vocab_size"], 70 + n) for n in (330, 150, 600)]
    ref = [P.forward(cfg, w, x).numpy() for x in ids]
    return d, ids, ref


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_big_layer_matches_plain(big_model, dtype):
    import janus_b200
    from janus_b200.engine import StepEntry
    from janus_b200.kernels import ops
    d, ids, ref = big_model
    model = janus_b200.load(d, dtype=dtype, max_tokens=1024)
    tol = tol_for(dtype)
    a, b = model.alloc_slot(), model.alloc_slot()
    # unequal prompts in one step; the first stops short of a page boundary (position 320)
    out = model.step([StepEntry(a, ids[0][:310], range(310)), StepEntry(b, ids[1][:100], range(100))]).cpu().numpy()
    assert rel_err(out[:310], ref[0][:310]) < tol and rel_err(out[310:], ref[1][:100]) < tol
    # one token each (CUDA-graph decode), across the boundary; the shorter sequence ends earlier
    rows_a, rows_b = [], []
    for j in range(20):
        entries = [StepEntry(a, [ids[0][310 + j]], [0])]
        if j < 12:
            entries.append(StepEntry(b, [ids[1][100 + j]], [0]))
        got = model.step(entries).cpu().numpy()
        rows_a.append(got[0:1])
        if j < 12:
            rows_b.append(got[1:2])
        if j == 11:
            model.free_slot(b)
    assert rel_err(np.concatenate(rows_a), ref[0][310:330]) < tol
    assert rel_err(np.concatenate(rows_b), ref[1][100:112]) < tol
    # the freed slot is used again: the rest of the second sequence from its start, in two chunks
    c = model.alloc_slot()
    first = model.step([StepEntry(c, ids[1][:64], [63])]).cpu().numpy()
    rest = model.step([StepEntry(c, ids[1][64:], range(86))]).cpu().numpy()
    assert rel_err(first, ref[1][63:64]) < tol and rel_err(rest, ref[1][64:]) < tol
    ops.check_kernel_status(model.device)


def test_long_prompt_runs_the_pair_products(big_model):
    import janus_b200
    from janus_b200.engine import StepEntry
    from janus_b200.kernels import ops
    d, ids, ref = big_model
    assert len(ids[2]) >= ops.QKV_FUSED_MIN_TOKENS
    model = janus_b200.load(d, dtype="bfloat16", max_tokens=1024)
    a = model.alloc_slot()
    out = model.step([StepEntry(a, ids[2], range(600))]).cpu().numpy()
    assert rel_err(out, ref[2]) < tol_for("bfloat16")
    ops.check_kernel_status(model.device)


@pytest.mark.parametrize("switch", ["fused_decode", "qkv_fused", "gemm_pair", "attn_tc"])
def test_the_documented_switches_select_kernels_that_give_the_same_logits(big_model, monkeypatch, switch):
    """JANUS_FUSED_DECODE=0, JANUS_QKV_FUSED=0, JANUS_GEMM_PAIR=0 and JANUS_ATTN_TC=0 each take a step through
    other kernels (rotation and append in a kernel of their own, a plain q/k/v projection, single-CTA
    products, mma.sync prompt attention); the environment is read at import, so the test turns the same
    module switches.  A prompt of 600 tokens, then tokens one by one."""
    import janus_b200
    from janus_b200.engine import StepEntry
    from janus_b200.kernels import ops
    from janus_b200.parts import attention
    d, ids, ref = big_model
    if switch == "fused_decode":
        monkeypatch.setattr(attention, "_FUSED_DECODE", False)
    elif switch == "qkv_fused":
        monkeypatch.setattr(ops, "_QKV_FUSED", False)
    elif switch == "gemm_pair":
        monkeypatch.setattr(ops, "_GEMM_PAIR", False)
    else:
        monkeypatch.setattr(ops, "_ATTN_TC", False)
    ops.gemm_plan.cache_clear()
    try:
        model = janus_b200.load(d, dtype="bfloat16", max_tokens=1024)
        a = model.alloc_slot()
        rows = [model.step([StepEntry(a, ids[2][:590], range(590))]).cpu().numpy()]
        for j in range(590, 600):
            rows.append(model.step([StepEntry(a, [ids[2][j]], [0])]).cpu().numpy())
        model.check()
        assert rel_err(np.concatenate(rows), ref[2]) < tol_for("bfloat16")
    finally:
        monkeypatch.undo()
        ops.gemm_plan.cache_clear()


def test_deterministic_mode_gives_the_same_bits_twice(big_model):
    """With the slices of a cut K summed in their fixed order nothing depends on the order of the day: two
    engines built one after the other give bitwise equal logits for a prompt and for decoded tokens."""
    import janus_b200
    from janus_b200.engine import StepEntry
    from janus_b200.kernels import ops
    d, ids, ref = big_model
    assert ops.split_k_for(8, 4096, 4096) > 1
    ops.set_deterministic(True)
    try:
        assert ops.split_k_for(8, 4096, 4096) > 1            # K is still cut; the sums are ordered
        runs = []
        for _ in range(2):
            model = janus_b200.load(d, dtype="bfloat16", max_tokens=1024)
            a = model.alloc_slot()
            rows = [model.step([StepEntry(a, ids[0][:300], range(300))]).cpu()]
            for j in range(300, 312):
                rows.append(model.step([StepEntry(a, [ids[0][j]], [0])]).cpu())
            runs.append(torch.cat(rows))
            model.check()
        assert torch.equal(runs[0], runs[1])
        assert rel_err(runs[0].numpy(), ref[0][:312]) < tol_for("bfloat16")
    finally:
        ops.set_deterministic(False)


# A context of several thousand keys: 71 pages a sequence, so that decode attention cuts its keys into
# splits that meet in the combine kernel, prompts run the products that work in CTA pairs and many row
# tiles of the tensor-core attention, and the llama3 frequency regions all occur among the positions.
LONG_CONTEXT = dict(
    architectures=["LlamaForCausalLM"], hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
    num_key_value_heads=2, head_dim=64, intermediate_size=512, vocab_size=512, max_position_embeddings=8192,
    rms_norm_eps=1e-5, rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=1024),
    tie_word_embeddings=True)
LONG_PROMPT, LONG_DECODED = 4500, 40


@pytest.fixture(scope="module")
def long_model(tmp_path_factory):
    d = make_model_dir(LONG_CONTEXT, str(tmp_path_factory.mktemp("long") / "m"), seed=5, dtype="bfloat16", sharpen=6.0)
    cfg, w = P.read_model_dir(d)
    ids = random_tokens(LONG_PROMPT + LONG_DECODED, LONG_CONTEXT["vocab_size"], 9)
    return d, ids, P.forward(cfg, w, ids).numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_context_of_thousands_of_keys(long_model, dtype):
    import janus_b200
    from janus_b200.engine import StepEntry
    d, ids, ref = long_model
    model = janus_b200.load(d, dtype=dtype, max_tokens=2 * 4608)
    tol = tol_for(dtype)
    a, b = model.alloc_slot(), model.alloc_slot()
    # the second sequence is a prefix of the first: its logits are the first's at the same places
    short = 1000
    want_a = list(range(0, LONG_PROMPT, 97)) + [LONG_PROMPT - 1]
    want_b = list(range(0, short, 89)) + [short - 1]
    out = model.step([StepEntry(a, ids[:LONG_PROMPT], want_a), StepEntry(b, ids[:short], want_b)]).cpu().numpy()
    assert rel_err(out[:len(want_a)], ref[want_a]) < tol
    assert rel_err(out[len(want_a):], ref[want_b]) < tol
    rows_a, rows_b = [], []
    for j in range(LONG_DECODED):
        got = model.step([StepEntry(a, [ids[LONG_PROMPT + j]], [0]), StepEntry(b, [ids[short + j]], [0])]).cpu().numpy()
        rows_a.append(got[0:1])
        rows_b.append(got[1:2])
    assert rel_err(np.concatenate(rows_a), ref[LONG_PROMPT:LONG_PROMPT + LONG_DECODED]) < tol
    assert rel_err(np.concatenate(rows_b), ref[short:short + LONG_DECODED]) < tol
    model.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_batch_of_a_hundred_sequences(tmp_path, dtype):
    """More sequences than any token tile of the decode products holds (64): a hundred prompts of 3 to 20
    tokens in one step, then five steps of one token each, every row against the plain implementation."""
    import janus_b200
    from janus_b200.engine import StepEntry
    from helpers import TINY_B
    d = make_model_dir(TINY_B, str(tmp_path / "m"), seed=3, dtype=dtype)
    cfg, w = P.read_model_dir(d)
    B = 100
    lens = [3 + (7 * i) % 18 for i in range(B)]
    ids = [random_tokens(n + 5, TINY_B["vocab_size"], 11 + i) for i, n in enumerate(lens)]
    ref = [P.forward(cfg, w, x).numpy() for x in ids]
    model = janus_b200.load(d, dtype=dtype, max_tokens=B * 64, max_slots=B)
    slots = [model.alloc_slot() for _ in range(B)]
    tol = tol_for(dtype)
    out = model.step([StepEntry(s, x[:n], [n - 1]) for s, x, n in zip(slots, ids, lens)]).cpu().numpy()
    assert rel_err(out, np.stack([r[n - 1] for r, n in zip(ref, lens)])) < tol
    for j in range(5):
        got = model.step([StepEntry(s, [x[n + j]], [0]) for s, x, n in zip(slots, ids, lens)]).cpu().numpy()
        assert rel_err(got, np.stack([r[n + j] for r, n in zip(ref, lens)])) < tol
    model.check()
