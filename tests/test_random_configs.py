"""Seeded random configurations of the architecture (head sizes from 16 to 256, groups that are no power of
two, widths and vocabularies that are no power of two, with and without rope scaling and a tied head), each
run through the engine in float32 and bfloat16 against the plain implementation: three prompts of unequal
length in one step (one of them long enough for the prompt-sized kernels), then token by token while the
shorter requests end."""
import random
import tempfile

import numpy as np
import pytest

import plain_llama as P
from helpers import make_model_dir, random_tokens, rel_err, tol_for

pytestmark = pytest.mark.gpu


def random_config(rng: random.Random) -> dict:
    nkv = rng.choice([1, 2, 3, 4])
    cfg = dict(architectures=["LlamaForCausalLM"],
               hidden_size=rng.choice([64, 72, 120, 200, 256, 320]),
               num_hidden_layers=rng.choice([1, 2, 3]),
               num_attention_heads=nkv * rng.choice([1, 2, 3, 4, 5, 8]),
               num_key_value_heads=nkv,
               head_dim=rng.choice([16, 24, 32, 40, 64, 64, 96, 128, 128, 256]),
               intermediate_size=rng.choice([104, 192, 320, 520]),
               vocab_size=rng.choice([131, 256, 300, 1000]),
               max_position_embeddings=1024,
               rms_norm_eps=rng.choice([1e-5, 1e-6]),
               rope_theta=rng.choice([10000.0, 500000.0]),
               tie_word_embeddings=rng.choice([True, False]))
    if rng.random() < 0.5:
        cfg["rope_scaling"] = dict(rope_type="llama3", factor=rng.choice([2.0, 8.0]), low_freq_factor=1.0,
                                   high_freq_factor=4.0, original_max_position_embeddings=rng.choice([32, 256]))
    return cfg


@pytest.mark.parametrize("seed", [11, 12, 13, 14, 15, 16])
def test_random_configuration_matches_plain(seed):
    import janus_b200
    from janus_b200.engine import StepEntry
    rng = random.Random(seed)
    cfg = random_config(rng)
    lens = [rng.randint(500, 900), rng.randint(1, 90), rng.randint(1, 400)]
    for dtype in ("float32", "bfloat16"):
        with tempfile.TemporaryDirectory() as d:
            make_model_dir(cfg, d, seed=seed, dtype=dtype, sharpen=1.5)
            c, w = P.read_model_dir(d)
            model = janus_b200.load(d, dtype=dtype, max_tokens=2048)
        ids = [random_tokens(n, cfg["vocab_size"], seed + n) for n in lens]
        ref = [P.forward(c, w, x).numpy() for x in ids]
        slots = [model.alloc_slot() for _ in ids]
        cut = [max(1, n - rng.randint(0, min(n - 1, 12))) for n in lens]
        out = model.step([StepEntry(s, x[:k], range(k)) for s, x, k in zip(slots, ids, cut)]).cpu().numpy()
        tol, start = tol_for(dtype), 0
        for i, k in enumerate(cut):
            assert rel_err(out[start:start + k], ref[i][:k]) < tol, (cfg, dtype, "prompt", i)
            start += k
        pos, rows = list(cut), [[] for _ in ids]
        while any(p < n for p, n in zip(pos, lens)):
            live = [i for i in range(len(ids)) if pos[i] < lens[i]]
            got = model.step([StepEntry(slots[i], [ids[i][pos[i]]], [0]) for i in live]).cpu().numpy()
            for r, i in enumerate(live):
                rows[i].append(got[r])
                pos[i] += 1
        for i in range(len(ids)):
            if rows[i]:
                assert rel_err(np.stack(rows[i]), ref[i][cut[i]:]) < tol, (cfg, dtype, "decode", i)
