"""The plain implementation checked against hand values (some from the
reference's own op tests, crates/janus-engine/src/compute/ops/tests.rs) and
against properties that follow from the formulas."""
import math

import torch

import plain_llama as P
from helpers import TINY_A, TINY_B, make_model_dir, random_tokens


def test_linear_hand_values():
    # ops/tests.rs:105-136: [[1,2,3],[4,5,6]] . [1,2,3] = [14, 32]
    w = torch.tensor([[1., 2., 3.], [4., 5., 6.]])
    assert P.linear(torch.tensor([[1., 2., 3.]]), w).tolist() == [[14., 32.]]


def test_rms_norm_hand_values():
    x = torch.tensor([[3., 4.]])
    y = P.rms_norm(x, torch.tensor([2., 0.5]), 0.0)
    rms = math.sqrt((9 + 16) / 2)
    assert torch.allclose(y, torch.tensor([[3 / rms * 2, 4 / rms * 0.5]]))
    assert float(P.rms_norm(torch.zeros(1, 4), torch.ones(4), 1e-5).abs().sum()) == 0.0


def test_rope_identity_at_zero_and_norm_preserving():
    # ops/tests.rs:334-390: position 0 leaves the vector unchanged
    x = torch.randn(3, 2, 16)
    inv = P.rope_inv_freq(16, 10000.0, None)
    cos, sin = P.rope_cos_sin(torch.zeros(3, dtype=torch.long), inv)
    assert torch.allclose(P.apply_rope(x, cos, sin), x)
    cos, sin = P.rope_cos_sin(torch.tensor([5, 17, 100]), inv)
    y = P.apply_rope(x, cos, sin)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    # pairs are (i, i + half): rotating a unit vector on axis 0 moves weight to axis 8 only
    e = torch.zeros(1, 1, 16); e[0, 0, 0] = 1.0
    r = P.apply_rope(e, *P.rope_cos_sin(torch.tensor([1]), inv))
    assert abs(float(r[0, 0, 0]) - math.cos(1.0)) < 1e-6 and abs(float(r[0, 0, 8]) - math.sin(1.0)) < 1e-6
    assert float(r[0, 0, 1:8].abs().sum() + r[0, 0, 9:].abs().sum()) == 0.0


def test_llama3_scaling_regions():
    s = TINY_B["rope_scaling"]
    base = P.rope_inv_freq(40, 500000.0, None)
    scaled = P.rope_inv_freq(40, 500000.0, s)
    wavelen = 2 * math.pi / base
    hi, lo = 32 / 4.0, 32 / 1.0
    assert torch.equal(scaled[wavelen < hi], base[wavelen < hi])                       # short waves kept
    assert torch.allclose(scaled[wavelen > lo], base[wavelen > lo] / 4.0)              # long waves slowed
    mid = (wavelen >= hi) & (wavelen <= lo)
    assert bool(mid.any()) and bool(((scaled[mid] <= base[mid]) & (scaled[mid] >= base[mid] / 4.0)).all())


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    q, k, v = torch.randn(6, 4, 8), torch.randn(6, 2, 8), torch.randn(6, 2, 8)
    out = P.attention(q, k, v)
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 3], v[0, 1])   # heads 0,1 -> kv 0; 2,3 -> kv 1
    k2, v2 = k.clone(), v.clone()
    k2[4:], v2[4:] = 9.0, 9.0
    assert torch.allclose(P.attention(q, k2, v2)[:4], out[:4])                          # the future changes nothing
    w = P.attention(q, k, v, window=2)
    s = (q[5, 0] @ k[4:6, 0].T) / math.sqrt(8)
    assert torch.allclose(w[5, 0], torch.softmax(s, 0) @ v[4:6, 0], atol=1e-6)


def test_sampling_functions():
    logits = torch.tensor([1.0, 3.0, 3.0, -2.0, 0.5])
    assert P.argmax_lowest(logits) == 1                                                # lowest index wins the tie
    assert P.apply_repetition_penalty(logits, [1, 3, 3], 2.0).tolist() == [1.0, 1.5, 3.0, -8.0, 0.5]
    tk = P.apply_top_k(logits, 3)
    assert tk.tolist()[:3] == [1.0, 3.0, 3.0] and tk[3] == float("-inf") and tk[4] == float("-inf")
    pr = P.softmax_probs(torch.tensor([0.0, float("-inf"), 0.0]))
    assert pr.tolist() == [0.5, 0.0, 0.5]
    tp = P.apply_top_p(torch.tensor([0.1, 0.5, 0.15, 0.25]), 0.7)
    assert torch.allclose(tp, torch.tensor([0.0, 0.5 / 0.75, 0.0, 0.25 / 0.75]))
    probs = torch.tensor([0.2, 0.3, 0.5])
    assert [P.sample_from_distribution(probs, u) for u in (0.0, 0.19, 0.21, 0.49, 0.51, 0.999)] == [0, 0, 1, 1, 2, 2]
    us = [P.uniform_for(1, r, s) for r in range(20) for s in range(20)]
    assert all(0.0 <= u < 1.0 for u in us) and len(set(us)) > 390 and abs(sum(us) / 400 - 0.5) < 0.06
    assert P.uniform_for(1, 2, 3) == P.uniform_for(1, 2, 3) != P.uniform_for(1, 3, 2)


def test_forward_prefix_property_and_schedule(tmp_path):
    d = make_model_dir(TINY_B, str(tmp_path / "b"), seed=1, dtype="float32")
    cfg, w = P.read_model_dir(d)
    ids = random_tokens(40, cfg["vocab_size"], 3)
    full = P.forward(cfg, w, ids)
    assert full.shape == (40, 384)
    assert torch.allclose(P.forward(cfg, w, ids[:17]), full[:17], atol=1e-5)            # causal: a prefix is a prefix
    assert "lm_head.weight" not in w                                                     # tied head
    twice = P.forward(cfg, w, ids, schedule=[0, 1, 1, 2])
    shared = P.forward(cfg, w, ids, schedule=[0, 1, (2, 1)])
    assert not torch.allclose(twice, full) and not torch.allclose(shared, full)
    out = P.generate(cfg, w, ids[:5], 6)
    assert len(out) == 6 and out[0] == P.argmax_lowest(P.forward(cfg, w, ids[:5])[-1])


def test_the_reference_s_own_op_cases():
    """Vectors of the reference's op tests, read from its source as text
    (crates/janus-engine/src/compute/ops/tests.rs:149-152 the matrix product with the second operand as [N, K];
    :403 and :430 the greedy pick on the GPU)."""
    a = torch.tensor([[1., 2., 3.], [4., 5., 6.]])
    b = torch.tensor([[7., 9., 11.], [8., 10., 12.]])
    assert P.linear(a, b).flatten().tolist() == [58., 64., 139., 154.]
    assert P.argmax_lowest(torch.tensor([-1.0, 0.5, 4.2, 3.9, 2.0])) == 2


def test_the_reference_s_own_sampler_cases():
    """The vectors of the reference's sampler tests, read from its source as text
    (crates/janus-engine/src/model/sampler.rs:871-891, 955-1000): the greedy pick, a NaN among the logits, and a
    batch of two rows with its default repetition penalty of 1.15 over the contexts [1, 2] and [5, 6]."""
    assert P.argmax_lowest(torch.tensor([0.1, 0.5, 0.3, 0.9, 0.2])) == 3
    assert P.argmax_lowest(torch.tensor([5.0, 1.0, 3.0])) == 0
    assert P.argmax_lowest(torch.tensor([-1.0, -5.0, -0.5])) == 2
    assert P.argmax_lowest(torch.tensor([0.1, float("nan"), 0.3, 0.2])) == 2
    rows = [[0.1, 0.2, 0.3, 0.9, 0.4, 0.1, 0.2, 0.1, 0.3, 0.2], [0.2, 0.1, 0.3, 0.2, 0.1, 0.4, 0.3, 0.8, 0.2, 0.1]]
    picks = [P.sample(torch.tensor(r), 0.0, 0.0, repetition_penalty=1.15, context=c)
             for r, c in zip(rows, ([1, 2], [5, 6]))]
    assert picks == [3, 7]
