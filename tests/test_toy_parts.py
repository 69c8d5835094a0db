"""Toy parts defined here, registered from here and run by the library's model,
step function and cache without a change to the library's files: a feed-forward
that routes every token to one of several experts, and a position encoding that
rotates neighbouring pairs.  They are no model of anyone's; they show that a
layer takes a part of another kind by its registered name, one layer at a time.
Each is compared with a plain restatement below: a prompt, unequal batches, one
token at a time, a slot used again."""
from dataclasses import replace

import pytest
import torch

import plain_llama as P
from helpers import TINY, random_tokens, rel_err, tol_for

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


# ---------------------------------------------------------------- a routed feed-forward
class ToyRoutedFeedForward:
    """Top-1 of `experts` gated feed-forwards; router logits in float32, lowest index on ties."""

    def __init__(self, hidden_size, intermediate_size, experts, dtype, device):
        self.H, self.I, self.E, self.dtype, self.device = hidden_size, intermediate_size, experts, dtype, device

    def weight_shapes(self):
        return {"router": ((self.E, self.H), "normal"),
                "w_in": ((self.E * 2 * self.I, self.H), "normal"),
                "w_out": ((self.E * self.H, self.I), "normal")}

    def load(self, router, w_in, w_out):
        self.router = router.to(self.device).float()
        self.w_in = w_in.to(self.device).float().view(self.E, 2 * self.I, self.H)
        self.w_out = w_out.to(self.device).float().view(self.E, self.H, self.I)

    def forward(self, x, residual, ctx):
        from janus_b200.kernels import ops
        xf = x.float()
        choice = torch.argmax(xf @ self.router.T, dim=-1)          # first maximum = lowest index
        out = torch.zeros_like(xf)
        for e in range(self.E):
            rows = torch.nonzero(choice == e).flatten()
            if rows.numel():
                gu = xf[rows] @ self.w_in[e].T
                g, u = gu[:, :self.I], gu[:, self.I:]
                out[rows] = (g * torch.sigmoid(g) * u) @ self.w_out[e].T
        ops.residual_add(residual, out.contiguous())


def plain_routed_ffn(x, router, w_in, w_out, E, I):
    H = x.shape[1]
    w_in, w_out = w_in.view(E, 2 * I, H), w_out.view(E, H, I)
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        logits = router @ x[t]
        e = int(torch.argmax(logits))
        gu = w_in[e] @ x[t]
        out[t] = w_out[e] @ (P.silu(gu[:I]) * gu[I:])
    return out


# ---------------------------------------------------------------- another position encoding
class ToyPairRotation:
    """Rotates the neighbouring pairs (2i, 2i+1) of every head by position * theta^(-2i/head_dim)."""

    def __init__(self, head_dim, theta, dtype, device):
        self.hd, self.theta, self.device = head_dim, theta, device
        self.inv = theta ** (-torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim)

    def weight_shapes(self):
        return {}

    def load(self):
        pass

    def fused_rotary_table(self):
        return None                     # not the half-split rotation the fused kernel knows: apply() is called

    def apply(self, x, heads, head_dim, positions):
        T = x.shape[0]
        ang = positions.float()[:, None] * self.inv[None, :]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        v = x.reshape(T, heads, head_dim // 2, 2).float()
        a, b = v[..., 0], v[..., 1]
        x.copy_(torch.stack([a * c - b * s, a * s + b * c], dim=-1).reshape(T, heads * head_dim))


def plain_pair_rotation(x, positions, theta):
    T, heads, hd = x.shape
    inv = theta ** (-torch.arange(0, hd, 2, dtype=torch.float32) / hd)
    ang = positions.float()[:, None] * inv[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    v = x.reshape(T, heads, hd // 2, 2)
    a, b = v[..., 0], v[..., 1]
    return torch.stack([a * c - b * s, a * s + b * c], dim=-1).reshape(T, heads, hd)


def plain_toy_forward(cfg, w, ids, E, I, theta, routed):
    """Layer 0: attention with the pair rotation, then the routed feed-forward (or the architecture's own);
    layer 1 as the architecture has it."""
    nh, nkv, hd = (P.cfg_get(cfg, k) for k in ("num_attention_heads", "num_key_value_heads", "head_dim"))
    eps = P.cfg_get(cfg, "rms_norm_eps")
    T = len(ids)
    pos = torch.arange(T)
    x = P.embed(w["model.embed_tokens.weight"], torch.tensor(ids))
    p = "model.layers.0."
    n = P.rms_norm(x, w[p + "input_layernorm.weight"], eps)
    q = plain_pair_rotation(P.linear(n, w[p + "self_attn.q_proj.weight"]).view(T, nh, hd), pos, theta)
    k = plain_pair_rotation(P.linear(n, w[p + "self_attn.k_proj.weight"]).view(T, nkv, hd), pos, theta)
    v = P.linear(n, w[p + "self_attn.v_proj.weight"]).view(T, nkv, hd)
    h1 = x + P.linear(P.attention(q, k, v).reshape(T, nh * hd), w[p + "self_attn.o_proj.weight"])
    n = P.rms_norm(h1, w[p + "post_attention_layernorm.weight"], eps)
    if routed:
        x = h1 + plain_routed_ffn(n, w["toy.router"], w["toy.w_in"], w["toy.w_out"], E, I)
    else:
        x = h1 + P.swiglu_ffn(n, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    x, _ = P.decoder_block(x, pos, cfg, w, 1)
    return P.linear(P.rms_norm(x, w["model.norm.weight"], eps), P.lm_head_weight(cfg, w))


# In 16 bits a token whose two best experts are nearly tied may go to the other one, which is no fault
# of the library: the routed feed-forward is compared in float32, the position encoding in both.
@pytest.mark.parametrize("dtype, routed", [("float32", True), ("float32", False), ("bfloat16", False)])
def test_toy_routing_and_toy_positions_register_build_and_step(dtype, routed):
    from janus_b200.config import LlamaConfig
    from janus_b200.engine import DecoderModel, Engine, EngineOptions, StepEntry
    from janus_b200.models.llama import llama_spec
    from janus_b200.parts import PartSpec, register_part
    from janus_b200.weights import RandomCheckpoint

    register_part("feed_forward", "toy_routed", ToyRoutedFeedForward)
    register_part("position", "toy_pair_rotation", ToyPairRotation)
    cfg = TINY["A"]
    E, I, theta = 3, 24, 100.0
    tdtype = getattr(torch, dtype)
    base = llama_spec(LlamaConfig.from_dict(cfg))
    mixer = base.layers[0].mixer
    toy_mixer = replace(mixer, params=dict(mixer.params, position=PartSpec("toy_pair_rotation",
                                                                            dict(head_dim=P.cfg_get(cfg, "head_dim"), theta=theta))))
    toy_ff = PartSpec("toy_routed", dict(hidden_size=cfg["hidden_size"], intermediate_size=I, experts=E),
                      weights=dict(router="toy.router", w_in="toy.w_in", w_out="toy.w_out"))
    layer0 = replace(base.layers[0], mixer=toy_mixer, feed_forward=toy_ff if routed else base.layers[0].feed_forward)
    spec = replace(base, layers=(layer0, base.layers[1]))
    model = DecoderModel(spec, tdtype, torch.device(DEV))
    names = [s.name for s in model.weight_specs()]
    assert ("toy.router" in names) == routed and any("layers.0.mlp" in n for n in names) != routed
    ck = RandomCheckpoint(model.weight_specs(), seed=9, dtype=dtype)
    model.load(ck)
    w = {n: ck.tensor(n).float() for n in ck.names()}
    eng = Engine(model, EngineOptions(max_tokens=512, max_slots=2, use_graphs=False))
    seqs = [random_tokens(n, cfg["vocab_size"], 60 + n) for n in (41, 12, 75)]
    ref = [plain_toy_forward(cfg, w, ids, E, I, theta, routed) for ids in seqs]
    tol = tol_for(dtype)
    s0, s1 = eng.alloc_slot(), eng.alloc_slot()
    a = eng.step([StepEntry(s0, seqs[0][:30], range(30)), StepEntry(s1, seqs[1][:7], range(7))]).cpu()
    assert rel_err(a[:30], ref[0][:30]) < tol and rel_err(a[30:], ref[1][:7]) < tol
    for j in range(5):
        b = eng.step([StepEntry(s0, [seqs[0][30 + j]], [0]), StepEntry(s1, [seqs[1][7 + j]], [0])]).cpu()
        assert rel_err(b[0:1], ref[0][30 + j:31 + j]) < tol and rel_err(b[1:2], ref[1][7 + j:8 + j]) < tol
    eng.free_slot(s1)
    c = eng.step([StepEntry(s0, seqs[0][35:], range(6))]).cpu()
    assert rel_err(c, ref[0][35:]) < tol
    s2 = eng.alloc_slot()
    d = eng.step([StepEntry(s2, seqs[2], range(75))]).cpu()
    assert rel_err(d, ref[2]) < tol


# ---------------------------------------------------------------- layers of another make
class ToySandwichBlock:
    """A toy arrangement with a part of its own: the mixer's output is normed once more before it joins the
    residual stream (h1 = x + post(mixer(pre(x)))), and the layer has no feed-forward at all.  The mixer adds
    into whatever float32 buffer it is handed, so it is handed a cleared one."""

    def __init__(self, parts, hidden_size, dtype):
        self.pre, self.mixer, self.post = parts["mixer_norm"], parts["mixer"], parts["post_mixer_norm"]
        assert "feed_forward" not in parts
        self.H, self.dtype = hidden_size, dtype

    def forward(self, residual, ctx, cache_view, writes_cache=True):
        from janus_b200.kernels import ops
        T = residual.shape[0]
        x = ctx.workspace.get("normed", (T, self.H), self.dtype)
        branch = ctx.workspace.get("toy_branch", (T, self.H), torch.float32)
        y = ctx.workspace.get("toy_branch_normed", (T, self.H), self.dtype)
        self.pre.forward(residual, x)
        branch.zero_()
        self.mixer.forward(x, branch, ctx, cache_view, writes_cache)
        self.post.forward(branch, y)
        ops.residual_add(residual, y)


class ToyScale:
    """A transform of a whole tensor in place: t *= factor (an embedding multiplier)."""

    def __init__(self, factor, dtype, device):
        self.factor = factor

    def weight_shapes(self):
        return {}

    def load(self):
        pass

    def forward(self, t, ctx):
        t.mul_(self.factor)


class ToySoftCap(ToyScale):
    """logits = cap * tanh(logits / cap)"""

    def forward(self, t, ctx):
        t.copy_(self.factor * torch.tanh(t / self.factor))


def plain_other_layers(cfg, w, ids, scale, cap):
    """Embedding times `scale`; layer 0: x + post_norm(attention(pre_norm(x))), no feed-forward; layer 1 as the
    architecture has it; logits soft-capped at `cap`."""
    eps = P.cfg_get(cfg, "rms_norm_eps")
    pos = torch.arange(len(ids))
    x = P.embed(w["model.embed_tokens.weight"], torch.tensor(ids)) * scale
    a, _ = P.attention_block(P.rms_norm(x, w["model.layers.0.input_layernorm.weight"], eps), pos, cfg, w, 0)
    x = x + P.rms_norm(a, w["toy.post_mixer_norm.weight"], eps)
    x, _ = P.decoder_block(x, pos, cfg, w, 1)
    logits = P.linear(P.rms_norm(x, w["model.norm.weight"], eps), P.lm_head_weight(cfg, w))
    return cap * torch.tanh(logits / cap)


@pytest.mark.parametrize("use_graphs", [False, True], ids=["no-graphs", "graphs"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_layer_without_feed_forward_an_arrangement_with_a_part_of_its_own_and_transforms(dtype, use_graphs):
    """What a layer consists of is data too: a layer may leave the feed-forward out, an arrangement registered
    from here takes a further norm by a role of its own, and transforms registered from here scale the
    embedding and cap the logits; the library's files stay as they are."""
    from janus_b200.config import LlamaConfig
    from janus_b200.engine import DecoderModel, Engine, EngineOptions, StepEntry
    from janus_b200.models.llama import llama_spec
    from janus_b200.parts import LayerSpec, PartSpec, register_part
    from janus_b200.weights import RandomCheckpoint

    register_part("arrangement", "toy_sandwich", ToySandwichBlock)
    register_part("transform", "toy_scale", ToyScale)
    register_part("transform", "toy_soft_cap", ToySoftCap)
    cfg = TINY["A"]
    scale, cap = 3.0, 0.4          # logits reach about 0.55: the cap bends them without flattening them
    base = llama_spec(LlamaConfig.from_dict(cfg))
    l0 = base.layers[0]
    post = PartSpec("rms_norm", dict(l0.mixer_norm.params), weights=dict(gamma="toy.post_mixer_norm.weight"))
    layer0 = LayerSpec(mixer=l0.mixer, mixer_norm=l0.mixer_norm, arrangement="toy_sandwich",
                       extra=(("post_mixer_norm", "norm", post),))
    spec = replace(base, layers=(layer0, base.layers[1]),
                   embedding_transforms=(PartSpec("toy_scale", dict(factor=scale)),),
                   logit_transforms=(PartSpec("toy_soft_cap", dict(factor=cap)),))
    model = DecoderModel(spec, getattr(torch, dtype), torch.device(DEV))
    names = [s.name for s in model.weight_specs()]
    assert "toy.post_mixer_norm.weight" in names and not any("layers.0.mlp" in n for n in names)
    assert not any("layers.0.post_attention_layernorm" in n for n in names)
    ck = RandomCheckpoint(model.weight_specs(), seed=12, dtype=dtype, norm_std=0.02)
    model.load(ck)
    w = {n: ck.tensor(n).float() for n in ck.names()}
    eng = Engine(model, EngineOptions(max_tokens=512, max_slots=2, use_graphs=use_graphs))
    seqs = [random_tokens(n, cfg["vocab_size"], 30 + n) for n in (80, 21)]
    ref = [plain_other_layers(cfg, w, ids, scale, cap) for ids in seqs]
    tol = tol_for(dtype)
    s0, s1 = eng.alloc_slot(), eng.alloc_slot()
    a = eng.step([StepEntry(s0, seqs[0][:50], range(50)), StepEntry(s1, seqs[1][:9], range(9))]).cpu()
    assert rel_err(a[:50], ref[0][:50]) < tol and rel_err(a[50:], ref[1][:9]) < tol
    for j in range(30):                                  # past position 64; the shorter sequence ends on the way
        entries = [StepEntry(s0, [seqs[0][50 + j]], [0])]
        if 9 + j < len(seqs[1]):
            entries.append(StepEntry(s1, [seqs[1][9 + j]], [0]))
        b = eng.step(entries).cpu()
        assert rel_err(b[0:1], ref[0][50 + j:51 + j]) < tol, f"position {50 + j}"
        if len(entries) == 2:
            assert rel_err(b[1:2], ref[1][9 + j:10 + j]) < tol


def test_an_arrangement_is_told_which_part_it_lacks():
    from janus_b200.config import LlamaConfig
    from janus_b200.engine import DecoderModel
    from janus_b200.models.llama import llama_spec
    from janus_b200.parts import LayerSpec
    base = llama_spec(LlamaConfig.from_dict(TINY["A"]))
    l0 = base.layers[0]
    with pytest.raises(ValueError, match="feed_forward_norm"):
        DecoderModel(replace(base, layers=(LayerSpec(mixer=l0.mixer, mixer_norm=l0.mixer_norm,
                                                     feed_forward=l0.feed_forward), base.layers[1])),
                     torch.float32, torch.device(DEV))


# ---------------------------------------------------------------- another norm
class ToyCenteredNorm:
    """A toy norm with two weights: y = (x - mean) / sqrt(var + eps) * gamma + beta, written with device
    operations of the tensor library (no kernel of this package)."""

    def __init__(self, width, eps, dtype, device):
        self.width, self.eps, self.dtype, self.device = width, eps, dtype, device

    def weight_shapes(self):
        return {"gamma": ((self.width,), "ones"), "beta": ((self.width,), "normal")}

    def load(self, gamma, beta):
        self.gamma, self.beta = gamma.to(self.device).float(), beta.to(self.device).float()

    def forward(self, x, out, row_index=None, clear=None):
        if clear is not None:
            clear.zero_()
        rows = x[:out.shape[0]] if row_index is None else x.index_select(0, row_index.long())
        mean = rows.mean(-1, keepdim=True)
        var = ((rows - mean) ** 2).mean(-1, keepdim=True)
        out.copy_((rows - mean) / torch.sqrt(var + self.eps) * self.gamma + self.beta)


def plain_centered(x, gamma, beta, eps):
    mean = x.mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(((x - mean) ** 2).mean(-1, keepdim=True) + eps) * gamma + beta


def plain_with_toy_norms(cfg, w, ids):
    """Layer 0 as the architecture has it; layer 1 and the model's last norm with the toy norm."""
    eps = 1e-3
    pos = torch.arange(len(ids))
    x = P.embed(w["model.embed_tokens.weight"], torch.tensor(ids))
    x, _ = P.decoder_block(x, pos, cfg, w, 0)
    a, _ = P.attention_block(plain_centered(x, w["toy.n1.gamma"], w["toy.n1.beta"], eps), pos, cfg, w, 1)
    x = x + a
    n = plain_centered(x, w["toy.n2.gamma"], w["toy.n2.beta"], eps)
    x = x + P.swiglu_ffn(n, w["model.layers.1.mlp.gate_proj.weight"], w["model.layers.1.mlp.up_proj.weight"],
                         w["model.layers.1.mlp.down_proj.weight"])
    return P.linear(plain_centered(x, w["toy.n3.gamma"], w["toy.n3.beta"], eps), P.lm_head_weight(cfg, w))


@pytest.mark.parametrize("use_graphs", [False, True], ids=["no-graphs", "graphs"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_toy_norm_with_two_weights_in_a_layer_and_before_the_head(dtype, use_graphs):
    """Another norm is a registry entry: a toy norm with a weight and a bias, defined here, norms both branches
    of layer 1 (where it also clears the mixer's scratch when asked) and the rows that go to the head (picked
    by `row_index`); layer 0 keeps the architecture's norm; the library's files stay as they are."""
    from janus_b200.config import LlamaConfig
    from janus_b200.engine import DecoderModel, Engine, EngineOptions, StepEntry
    from janus_b200.models.llama import llama_spec
    from janus_b200.parts import PartSpec, register_part
    from janus_b200.weights import RandomCheckpoint

    register_part("norm", "toy_centered", ToyCenteredNorm)
    cfg = TINY["A"]
    base = llama_spec(LlamaConfig.from_dict(cfg))

    def toy(tag):
        return PartSpec("toy_centered", dict(width=cfg["hidden_size"], eps=1e-3),
                        weights=dict(gamma=f"toy.{tag}.gamma", beta=f"toy.{tag}.beta"))

    layer1 = replace(base.layers[1], mixer_norm=toy("n1"), feed_forward_norm=toy("n2"))
    spec = replace(base, layers=(base.layers[0], layer1), final_norm=toy("n3"))
    model = DecoderModel(spec, getattr(torch, dtype), torch.device(DEV))
    names = [s.name for s in model.weight_specs()]
    assert "toy.n3.beta" in names and "model.norm.weight" not in names
    assert not any("layers.1.input_layernorm" in n or "layers.1.post_attention_layernorm" in n for n in names)
    ck = RandomCheckpoint(model.weight_specs(), seed=14, dtype=dtype, norm_std=0.05)
    model.load(ck)
    w = {n: ck.tensor(n).float() for n in ck.names()}
    eng = Engine(model, EngineOptions(max_tokens=512, max_slots=2, use_graphs=use_graphs))
    seqs = [random_tokens(n, cfg["vocab_size"], 90 + n) for n in (75, 20)]
    ref = [plain_with_toy_norms(cfg, w, ids) for ids in seqs]
    tol = tol_for(dtype)
    s0, s1 = eng.alloc_slot(), eng.alloc_slot()
    a = eng.step([StepEntry(s0, seqs[0][:40], [0, 17, 39]), StepEntry(s1, seqs[1][:9], [8])]).cpu()
    assert rel_err(a[:3], ref[0][[0, 17, 39]]) < tol and rel_err(a[3:], ref[1][8:9]) < tol
    for j in range(30):                                  # past position 64; the shorter sequence ends on the way
        entries = [StepEntry(s0, [seqs[0][40 + j]], [0])]
        if 9 + j < len(seqs[1]):
            entries.append(StepEntry(s1, [seqs[1][9 + j]], [0]))
        b = eng.step(entries).cpu()
        assert rel_err(b[0:1], ref[0][40 + j:41 + j]) < tol, f"position {40 + j}"
        if len(entries) == 2:
            assert rel_err(b[1:2], ref[1][9 + j:10 + j]) < tol
