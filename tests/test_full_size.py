"""The Llama-3.1-8B shape at its real sizes: two layers with the real vocabulary of 128,256 against the plain
implementation, and all 32 layers in bfloat16 against the true 32-bit engine on the same weights.  The weights
are the seeded random ones that `bench.py` times; they are made on the device and, bit for bit the same, for
the oracle."""
import numpy as np
import pytest
import torch

import plain_llama as P
from helpers import BF16_TOL, FP32_TOL, random_tokens, rel_err

pytestmark = pytest.mark.gpu

CONFIG_8B = dict(
    architectures=["LlamaForCausalLM"], hidden_size=4096, num_hidden_layers=32, num_attention_heads=32,
    num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=128256,
    max_position_embeddings=4096, rms_norm_eps=1e-5, rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=8192),
    tie_word_embeddings=False)
PROMPT, DECODED = 96, 8


def drive(model, ids, want):
    """A prompt in one step with the logits of the places `want`, then single tokens."""
    from janus_b200.engine import StepEntry
    s = model.alloc_slot()
    rows = [model.step([StepEntry(s, ids[:PROMPT], want)]).cpu().numpy()]
    for j in range(PROMPT, PROMPT + DECODED):
        rows.append(model.step([StepEntry(s, [ids[j]], [0])]).cpu().numpy())
    model.check()
    model.free_slot(s)
    return np.concatenate(rows)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_layers_with_the_real_vocabulary_match_plain(dtype):
    """The head over 128,256 rows (1,002 row tiles of 128 and a ragged last one) and the embedding at its
    real size, which no small configuration reaches."""
    import janus_b200
    from janus_b200.config import resolve_architecture
    from janus_b200.weights import RandomCheckpoint
    cfg = dict(CONFIG_8B, num_hidden_layers=2)
    arch = resolve_architecture(cfg)
    # the oracle's weights: the same seeded source, made on the device (same bits as on the host), in float32 on the CPU
    ck = RandomCheckpoint(arch.weight_specs(arch.config_class.from_dict(cfg)), 2, dtype=dtype, std=0.02,
                          norm_std=0.02, device="cuda:0")
    w = {n: ck.tensor(n).float().cpu() for n in ck.names()}
    ids = random_tokens(PROMPT + DECODED, cfg["vocab_size"], 77)
    ids[5], ids[40] = cfg["vocab_size"] - 1, 0                  # the last and the first row of the table
    want = [0, 5, 40, 63, 64, PROMPT - 1]
    ref = P.forward(cfg, w, ids).numpy()[want + list(range(PROMPT, PROMPT + DECODED))]
    del w
    model = janus_b200.load_random(cfg, seed=2, dtype=dtype, max_tokens=256, max_slots=2, std=0.02, norm_std=0.02)
    got = drive(model, ids, want)
    assert got.shape == (len(want) + DECODED, cfg["vocab_size"])
    assert rel_err(got, ref) < (FP32_TOL if dtype == "float32" else BF16_TOL)
    # the ragged end of the vocabulary: the last row tile holds 128256 - 1001 * 128 = 128 rows here, so also
    # look at the extremes by name
    assert np.abs(got[:, -1] - ref[:, -1]).max() < BF16_TOL * np.abs(ref).max()


# What bfloat16 costs per layer.  A bfloat16 value keeps 8 bits of mantissa: rounding moves it by up to 2^-8 of
# its binade, about 0.16 % rms.  A layer rounds its normed input (twice), q, k, v, the softmax weights, the
# attention output and the gated activation; a score q.k carries the errors of both operands and of the normed
# input behind each, about 0.5 % per key.  Together about 0.8 % of a layer's output, which is what one layer of
# these sizes measures (0.78 % rms of the logits against the 32-bit engine; 1.0 % at 2 layers, 2.0 % at 8, 4.0 %
# at 32).  Layers are independent, so the error grows like the square root of the depth, as the signal does not:
# the bound is BF16_LAYER_ERR * sqrt(layers), with a third of head-room over the measured 0.78 %.
BF16_LAYER_ERR = 1.1e-2


def rms_err(got, ref):
    got, ref = got.astype(np.float64), ref.astype(np.float64)
    assert np.isfinite(got).all()
    return float(np.sqrt(((got - ref) ** 2).mean()) / np.sqrt((ref ** 2).mean()))


def test_all_32_layers_in_bfloat16_against_the_32_bit_engine():
    """Full depth, the weights of the benchmark (seed 2), the bfloat16 engine against the true 32-bit engine on
    the same (bfloat16-valued) weights: a prompt of 96 tokens, then 8 tokens one by one.  The error must stay
    within the rounding budget of 32 layers, and it must have grown from 8 layers to 32 as a random walk does
    (twice; a fault in one deep layer, or an offset that overflows with depth, breaks the ratio long before it
    breaks the budget).  Where the 32-bit engine's best logit leads clearly, both choose the same token."""
    import janus_b200
    ids = random_tokens(PROMPT + DECODED, CONFIG_8B["vocab_size"], 78)
    want = [0, 31, 64, PROMPT - 1]
    errs = {}
    for layers in (8, 32):
        outs = {}
        for dtype in ("float32", "bfloat16"):
            model = janus_b200.load_random(dict(CONFIG_8B, num_hidden_layers=layers), seed=2, dtype=dtype,
                                           max_tokens=256, max_slots=2, std=0.02, norm_std=0.0,
                                           stored_dtype="bfloat16")
            outs[dtype] = drive(model, ids, want)
            del model
            torch.cuda.empty_cache()
        errs[layers] = rms_err(outs["bfloat16"], outs["float32"])
        print(f"bfloat16 against float32 over {layers} layers: {errs[layers]:.4f} rms of the logits' rms")
        assert errs[layers] < BF16_LAYER_ERR * layers ** 0.5
    assert errs[32] < 1.5 * 2.0 * errs[8]
    f, b = outs["float32"], outs["bfloat16"]
    top2 = np.sort(f, axis=1)[:, -2:]
    clear = (top2[:, 1] - top2[:, 0]) > 6 * errs[32] * float(np.sqrt((f.astype(np.float64) ** 2).mean()))
    assert (f.argmax(1)[clear] == b.argmax(1)[clear]).all()


def test_a_prompt_of_24000_tokens_in_bfloat16_chunks_against_the_32_bit_engine_in_one_step():
    """A long sequence through the whole engine: 375 pages, rotation angles at positions far beyond the small
    tests', the prompt cut into four steps of 6,000 tokens for the bfloat16 engine (prompt attention over a cache
    that earlier steps left) and run as one step by the 32-bit engine, then three tokens one by one.  The logits
    at the ends of the chunks, at the prompt's last tokens and at the decoded ones agree within the rounding of
    two layers."""
    import janus_b200
    from janus_b200.engine import StepEntry
    cfg = dict(architectures=["LlamaForCausalLM"], hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, head_dim=64, intermediate_size=640, vocab_size=1000,
               max_position_embeddings=32768, rms_norm_eps=1e-5, rope_theta=500000.0,
               rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                 original_max_position_embeddings=8192),
               tie_word_embeddings=True)
    n, chunk = 24000, 6000
    ids = random_tokens(n + 3, cfg["vocab_size"], 79)
    ends = [chunk - 1, 2 * chunk - 1, 3 * chunk - 1, n - 2, n - 1]
    outs = {}
    for dtype in ("float32", "bfloat16"):
        model = janus_b200.load_random(cfg, seed=5, dtype=dtype, max_tokens=n + 64, max_slots=1, std=0.05,
                                       norm_std=0.02, stored_dtype="bfloat16")
        s = model.alloc_slot()
        rows = []
        if dtype == "float32":
            rows.append(model.step([StepEntry(s, ids[:n], ends)]).cpu().numpy())
        else:
            for c in range(0, n, chunk):
                want = [e - c for e in ends if c <= e < c + chunk]
                rows.append(model.step([StepEntry(s, ids[c:c + chunk], want)]).cpu().numpy())
        for j in range(n, n + 3):
            rows.append(model.step([StepEntry(s, [ids[j]], [0])]).cpu().numpy())
        model.check()
        model.free_slot(s)
        outs[dtype] = np.concatenate(rows)
        del model
        torch.cuda.empty_cache()
    assert outs["float32"].shape == (len(ends) + 3, cfg["vocab_size"])
    err = rms_err(outs["bfloat16"], outs["float32"])
    print(f"24,000 tokens, bfloat16 in chunks against float32 whole: {err:.4f} rms of the logits' rms")
    assert err < BF16_LAYER_ERR * 2 ** 0.5
