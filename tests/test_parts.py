"""Each part of a layer alone against its plain counterpart, a schedule that
names a layer twice or reads another layer's cache, and a toy mixer with state
of its own that is registered, built and stepped from here, without a change to
the library's files."""
import math

import pytest
import torch

import plain_llama as P
from helpers import TINY, make_model_dir, random_tokens, rel_err, tol_for

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def load(tmp_path, name, dtype, **kw):
    import janus_b200
    d = make_model_dir(TINY[name], str(tmp_path / f"m{name}{dtype}"), seed=4, dtype=dtype)
    return janus_b200.load(d, dtype=dtype, max_tokens=1024, use_graphs=False, **kw), P.read_model_dir(d)


def context(model, ids):
    from janus_b200.engine.step import StepEntry
    eng = model.engine
    slot = eng.alloc_slot()
    entries = [StepEntry(slot, ids, ())]
    eng._reserve(entries)
    ctx, _, _ = eng.build_context(entries)
    return ctx


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_parts_alone(tmp_path, name, dtype):
    model, (cfg, w) = load(tmp_path, name, dtype)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    tol = tol_for(dtype)
    T, H = 77, cfg["hidden_size"]
    ids = random_tokens(T, cfg["vocab_size"], 9)
    ctx = context(model, ids)
    layer = model.engine.model.layers[1]
    g = torch.Generator().manual_seed(1)
    x = torch.randn(T, H, generator=g).to(tdt)               # a normed layer input, exact in the engine dtype
    res0 = torch.randn(T, H, generator=g)
    pos = torch.arange(T)
    # norm
    out = torch.empty(T, H, device=DEV, dtype=tdt)
    layer.mixer_norm.forward(res0.to(DEV), out)
    assert rel_err(out.float().cpu(), P.rms_norm(res0, w["model.layers.1.input_layernorm.weight"],
                                                 P.cfg_get(cfg, "rms_norm_eps"))) < tol
    # mixer (attention with rotary positions and the cache) adds into the residual
    res = res0.clone().to(DEV)
    layer.mixer.forward(x.to(DEV), res, ctx, ctx.cache_view(1), True)
    a, (k_rot, v) = P.attention_block(x.float(), pos, cfg, w, 1)
    assert rel_err((res.cpu() - res0), a) < tol
    # what it left in the cache: rotated keys, raw values, at the sequence's rows
    view = ctx.cache_view(1)
    rows = view.group.dest_rows.cpu().long()
    kc = view.k.float().cpu()[rows // 64, :, rows % 64, :]
    vc = view.v.float().cpu()[rows // 64, :, rows % 64, :]
    assert rel_err(kc, k_rot) < tol and rel_err(vc, v) < tol
    # feed-forward
    res = res0.clone().to(DEV)
    layer.feed_forward.forward(x.to(DEV), res, ctx)
    p = "model.layers.1.mlp."
    f = P.swiglu_ffn(x.float(), w[p + "gate_proj.weight"], w[p + "up_proj.weight"], w[p + "down_proj.weight"])
    assert rel_err(res.cpu() - res0, f) < tol
    # the arrangement: a whole block on the residual stream
    res = res0.clone().to(DEV)
    model.engine.model.layers[0].forward(res, ctx, ctx.cache_view(0), True)
    want, _ = P.decoder_block(res0, pos, cfg, w, 0)
    assert rel_err(res.cpu(), want) < tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_schedule_is_data(tmp_path, dtype):
    """Layer 1 runs twice; then a place reads the keys and values of an earlier place."""
    import janus_b200
    from dataclasses import replace
    from janus_b200.config import LlamaConfig
    from janus_b200.engine import DecoderModel, Engine, EngineOptions, StepEntry
    from janus_b200.models.llama import llama_spec
    from janus_b200.parts import ScheduleEntry
    from janus_b200.weights import FolderCheckpoint

    d = make_model_dir(TINY["B"], str(tmp_path / "m"), seed=2, dtype=dtype)
    cfg, w = P.read_model_dir(d)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    ids = random_tokens(90, cfg["vocab_size"], 1)
    for schedule, plain_schedule in (
            ((ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(1), ScheduleEntry(2)), [0, 1, 1, 2]),
            ((ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2, reads_cache_of=1)), [0, 1, (2, 1)])):
        spec = replace(llama_spec(LlamaConfig.from_dict(TINY["B"])), schedule=schedule)
        m = DecoderModel(spec, tdt, torch.device(DEV))
        m.load(FolderCheckpoint(d))
        eng = Engine(m, EngineOptions(max_tokens=256, use_graphs=False))
        s = eng.alloc_slot()
        first = eng.step([StepEntry(s, ids[:50], range(50))]).cpu()
        rest = torch.cat([eng.step([StepEntry(s, [t], [0])]).cpu() for t in ids[50:]])
        ref = P.forward(cfg, w, ids, schedule=plain_schedule)
        assert rel_err(torch.cat([first, rest]), ref) < tol_for(dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_with_and_without_a_window_have_storage_of_their_own(tmp_path, dtype):
    """Layer 0 keeps all keys, layers 1 and 2 only the last 70: two cache groups; the window
    group gives back the pages its queries have passed, and the logits match the plain model
    at the window's edge, for a prompt cut into steps and decoded past several pages."""
    from dataclasses import replace
    from janus_b200.config import LlamaConfig
    from janus_b200.engine import DecoderModel, Engine, EngineOptions, StepEntry
    from janus_b200.models.llama import llama_spec
    from janus_b200.parts import PartSpec
    from janus_b200.weights import FolderCheckpoint

    window = 70
    d = make_model_dir(TINY["B"], str(tmp_path / "m"), seed=5, dtype=dtype)
    cfg, w = P.read_model_dir(d)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    base = llama_spec(LlamaConfig.from_dict(TINY["B"]))
    layers = [base.layers[0]] + [
        replace(l, mixer=PartSpec(l.mixer.kind, dict(l.mixer.params, window=window), l.mixer.weights))
        for l in base.layers[1:]]
    m = DecoderModel(replace(base, layers=tuple(layers)), tdt, torch.device(DEV))
    m.load(FolderCheckpoint(d))
    eng = Engine(m, EngineOptions(max_tokens=512, use_graphs=(dtype == "bfloat16")))
    assert len(eng.cache.groups) == 2 and sorted(g.spec.window for g in eng.cache.groups) == [0, window]
    ids = random_tokens(230, cfg["vocab_size"], 6)

    def plain(ids):      # the plain model with a window on layers 1 and 2
        x = P.embed(w["model.embed_tokens.weight"], torch.tensor(ids))
        pos = torch.arange(len(ids))
        for layer in range(3):
            x, _ = P.decoder_block(x, pos, cfg, w, layer, window=None if layer == 0 else window)
        z = P.rms_norm(x, w["model.norm.weight"], P.cfg_get(cfg, "rms_norm_eps"))
        return P.linear(z, P.lm_head_weight(cfg, w))

    ref = plain(ids)
    s = eng.alloc_slot()
    got = [eng.step([StepEntry(s, ids[:100], range(100))]).cpu(), eng.step([StepEntry(s, ids[100:150], range(50))]).cpu()]
    got += [eng.step([StepEntry(s, [t], [0])]).cpu() for t in ids[150:]]
    assert rel_err(torch.cat(got), ref) < tol_for(dtype)
    full, win = sorted(eng.cache.groups, key=lambda g: g.spec.window)
    assert full.pool.n_held == 4 and win.pool.n_held <= 3           # 230 tokens: 4 pages; a window of 70 spans at most 3
    assert win.pages[s][0] == -1 and win.pages[s][1] == -1
    eng.free_slot(s)
    eng.cache.check()
    assert full.pool.n_held == 0 and win.pool.n_held == 0


class RunningMeanMixer:
    """Toy mixer with fixed-size state: out_t = scale * mean(x_0 .. x_t) over the
    sequence so far.  State per sequence: the running sum (H floats) and the count.
    Device work only, on the current stream, so that a decode step can be recorded
    into a CUDA graph and replayed."""

    def __init__(self, hidden_size, scale, dtype, device):
        self.H, self.scale, self.dtype, self.device = hidden_size, scale, dtype, device

    def weight_shapes(self):
        return {}

    def load(self):
        pass

    def cache_spec(self):
        from janus_b200.parts import StateSpec
        return StateSpec((self.H + 1,))

    def forward(self, x, residual, ctx, cache_view, writes_cache=True):
        from janus_b200.kernels import ops
        H, state = self.H, cache_view.state                      # [slots, H + 1]
        seq = ctx.token_seq.long()                               # sequence of each token
        slots = ctx.seq_slot.long()
        starts = ctx.q_start.long()
        xf = x.float()
        total = torch.cumsum(xf, 0)
        before = torch.cat([torch.zeros(1, H, device=x.device), total])[starts[:-1]]    # sum ahead of each sequence
        prev = state[slots]
        csum = total - before[seq] + prev[seq, :H]
        count = prev[seq, H] + (torch.arange(x.shape[0], device=x.device) - starts[:-1][seq] + 1)
        last = starts[1:] - 1
        state.index_copy_(0, slots, torch.cat([csum[last], count[last, None]], dim=1))
        ops.residual_add(residual, (self.scale * csum / count[:, None]).contiguous())


def plain_toy_forward(cfg, w, ids, scale):
    """Layer 0 with the running-mean mixer, layer 1 as the architecture has it."""
    x = P.embed(w["model.embed_tokens.weight"], torch.tensor(ids))
    pos = torch.arange(len(ids))
    eps = P.cfg_get(cfg, "rms_norm_eps")
    n = P.rms_norm(x, w["model.layers.0.input_layernorm.weight"], eps)
    h1 = x + scale * torch.cumsum(n, 0) / torch.arange(1, len(ids) + 1)[:, None]
    p = "model.layers.0."
    x = h1 + P.swiglu_ffn(P.rms_norm(h1, w[p + "post_attention_layernorm.weight"], eps),
                          w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    x, _ = P.decoder_block(x, pos, cfg, w, 1)
    return P.linear(P.rms_norm(x, w["model.norm.weight"], eps), P.lm_head_weight(cfg, w))


def toy_state_engine(use_graphs):
    from dataclasses import replace
    from janus_b200.config import LlamaConfig
    from janus_b200.engine import DecoderModel, Engine, EngineOptions
    from janus_b200.models.llama import llama_spec
    from janus_b200.parts import PartSpec, register_part
    from janus_b200.weights import RandomCheckpoint

    register_part("mixer", "toy_running_mean", RunningMeanMixer)
    cfg = TINY["A"]
    base = llama_spec(LlamaConfig.from_dict(cfg))
    toy_layer = replace(base.layers[0], mixer=PartSpec("toy_running_mean", dict(hidden_size=64, scale=0.5)))
    spec = replace(base, layers=(toy_layer, base.layers[1]))
    model = DecoderModel(spec, torch.float32, torch.device(DEV))
    names = [s.name for s in model.weight_specs()]
    assert not any("layers.0.self_attn" in n for n in names) and any("layers.1.self_attn" in n for n in names)
    ck = RandomCheckpoint(model.weight_specs(), seed=8, dtype="float32")
    model.load(ck)
    w = {n: ck.tensor(n) for n in ck.names()}
    return Engine(model, EngineOptions(max_tokens=512, max_slots=2, use_graphs=use_graphs)), cfg, w


@pytest.mark.parametrize("use_graphs", [False, True], ids=["no-graphs", "graphs"])
def test_toy_mixer_with_state_registers_builds_and_steps(use_graphs):
    from janus_b200.engine import StepEntry
    eng, cfg, w = toy_state_engine(use_graphs)
    seqs = [random_tokens(n, 256, 40 + n) for n in (37, 9, 70)]
    ref = [plain_toy_forward(cfg, w, ids, 0.5) for ids in seqs]
    # two sequences together: prompts of unequal length, then one token each
    s0, s1 = eng.alloc_slot(), eng.alloc_slot()
    a = eng.step([StepEntry(s0, seqs[0][:20], range(20)), StepEntry(s1, seqs[1][:5], range(5))]).cpu()
    assert rel_err(a[:20], ref[0][:20]) < 1e-4 and rel_err(a[20:], ref[1][:5]) < 1e-4
    for j in range(4):
        b = eng.step([StepEntry(s0, [seqs[0][20 + j]], [0]), StepEntry(s1, [seqs[1][5 + j]], [0])]).cpu()
        assert rel_err(b[0:1], ref[0][20 + j:21 + j]) < 1e-4 and rel_err(b[1:2], ref[1][5 + j:6 + j]) < 1e-4
    eng.free_slot(s1)
    c = eng.step([StepEntry(s0, seqs[0][24:], range(13))]).cpu()
    assert rel_err(c, ref[0][24:]) < 1e-4
    # the freed slot is used again; its state starts from zero
    s2 = eng.alloc_slot()
    assert s2 == s1
    d = eng.step([StepEntry(s2, seqs[2], range(70))]).cpu()
    assert rel_err(d, ref[2]) < 1e-4


def test_state_is_stepped_once_by_every_decode_step_under_cuda_graphs():
    """Decode steps replay CUDA graphs; a step that finds no graph (a new batch size, a page capacity that a
    sequence outgrew) must still advance a mixer's state exactly once.  Two sequences decode token by token
    from short prompts past position 64 (the page capacity doubles), the shorter one ends on the way (the
    batch size changes); every row is compared with the plain restatement."""
    from janus_b200.engine import StepEntry
    eng, cfg, w = toy_state_engine(True)
    seqs = [random_tokens(n, 256, 90 + n) for n in (120, 50)]
    ref = [plain_toy_forward(cfg, w, ids, 0.5) for ids in seqs]
    s0, s1 = eng.alloc_slot(), eng.alloc_slot()
    eng.step([StepEntry(s0, seqs[0][:20], ()), StepEntry(s1, seqs[1][:7], ())])
    pos = [20, 7]
    captures = eng.graph_captures
    while pos[0] < len(seqs[0]):
        live = [i for i in (0, 1) if pos[i] < len(seqs[i])]
        out = eng.step([StepEntry((s0, s1)[i], [seqs[i][pos[i]]], [0]) for i in live]).cpu()
        for row, i in enumerate(live):
            err = rel_err(out[row:row + 1], ref[i][pos[i]:pos[i] + 1])
            assert err < 1e-4, f"sequence {i} at position {pos[i]}: {err}"
            pos[i] += 1
    # batch of two at capacity 1, then one sequence at capacities 1 and 2
    assert eng.graph_captures - captures >= 3
