"""A whole toy architecture, defined and registered here: a configuration class with key names of its own, a
function from it to a `ModelSpec` (layers with and without a window, a place of the schedule that runs a layer a
second time on the cache the first run wrote, tensor names of its own, a tied head), and one registry entry.
The folder writer, the loader, the cache, the step function, the generation loop and the sampler then serve it
through the public entry points as they serve the Llama decoder; none of the library's files knows it.  It is a
test object and no model of anyone's."""
from dataclasses import asdict, dataclass
from typing import Tuple

import pytest
import torch

import plain_llama as P
from helpers import BF16_TOL, random_tokens, rel_err, tol_for

pytestmark = pytest.mark.gpu
NAME = "ToyWindowedDecoderForTest"


@dataclass(frozen=True)
class ToyConfig:
    width: int
    depth: int
    heads: int
    groups: int                  # key/value heads
    head_size: int
    inner: int
    vocab: int
    positions: int
    eps: float
    base: float
    window: int                  # odd layers see this many keys
    end_tokens: Tuple[int, ...] = ()
    architectures: Tuple[str, ...] = (NAME,)

    @classmethod
    def from_dict(cls, d):
        from janus_b200.config import ConfigError
        try:
            c = cls(**{k: (tuple(v) if isinstance(v, list) else v) for k, v in d.items() if k != "torch_dtype"})
        except TypeError as e:
            raise ConfigError(f"toy configuration: {e}") from None
        if c.heads % c.groups:
            raise ConfigError(f"key 'heads' ({c.heads}) must be divisible by 'groups' ({c.groups})")
        return c

    def to_dict(self):
        return {k: (list(v) if isinstance(v, tuple) else v) for k, v in asdict(self).items()}

    def stop_token_ids(self):
        return self.end_tokens


def toy_spec(c: ToyConfig):
    from janus_b200.parts import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    position = PartSpec("rotary", dict(head_dim=c.head_size, theta=c.base, max_positions=c.positions, scaling=None))
    layers = []
    for i in range(c.depth):
        p = f"blocks.{i}."
        layers.append(LayerSpec(
            mixer=PartSpec("gqa_attention", dict(hidden_size=c.width, num_heads=c.heads, num_kv_heads=c.groups,
                                                 head_dim=c.head_size, position=position,
                                                 window=c.window if i % 2 else 0),
                           weights=dict(q=p + "attn.wq", k=p + "attn.wk", v=p + "attn.wv", o=p + "attn.wo")),
            feed_forward=PartSpec("swiglu", dict(hidden_size=c.width, intermediate_size=c.inner),
                                  weights=dict(gate=p + "ff.w1", up=p + "ff.w3", down=p + "ff.w2")),
            mixer_norm=PartSpec("rms_norm", dict(width=c.width, eps=c.eps), weights=dict(gamma=p + "norm_a")),
            feed_forward_norm=PartSpec("rms_norm", dict(width=c.width, eps=c.eps), weights=dict(gamma=p + "norm_f"))))
    # every layer once, then layer 1 once more on the keys and values its first run wrote
    schedule = tuple(ScheduleEntry(i) for i in range(c.depth)) + (ScheduleEntry(1, reads_cache_of=1),)
    return ModelSpec(hidden_size=c.width, vocab_size=c.vocab, layers=tuple(layers), schedule=schedule,
                     final_norm=PartSpec("rms_norm", dict(width=c.width, eps=c.eps), weights=dict(gamma="out_norm")),
                     embedding_weight="tokens.table", head_weight=None, max_positions=c.positions)


def register():
    from janus_b200.config import register_architecture
    from janus_b200.engine.model import DecoderModel, model_weight_specs
    register_architecture(NAME, ToyConfig, lambda c, dtype, device: DecoderModel(toy_spec(c), dtype, device),
                          lambda c: model_weight_specs(toy_spec(c)))


TOY = dict(architectures=[NAME], width=96, depth=3, heads=6, groups=2, head_size=24, inner=200, vocab=311,
           positions=256, eps=1e-5, base=5000.0, window=40, end_tokens=[310])


def plain_toy(c: ToyConfig, w, ids):
    """The same model from the plain implementation's parts: the toy's tensors under the names those parts
    look up, a window on the odd layers, layer 1 a second time at the end on its first run's keys and values."""
    cfg = dict(hidden_size=c.width, num_hidden_layers=c.depth, num_attention_heads=c.heads,
               num_key_value_heads=c.groups, head_dim=c.head_size, intermediate_size=c.inner, vocab_size=c.vocab,
               rms_norm_eps=c.eps, rope_theta=c.base, tie_word_embeddings=True)
    m = {"model.embed_tokens.weight": w["tokens.table"], "model.norm.weight": w["out_norm"]}
    for i in range(c.depth):
        a, b = f"blocks.{i}.", f"model.layers.{i}."
        for toy, llama in (("attn.wq", "self_attn.q_proj.weight"), ("attn.wk", "self_attn.k_proj.weight"),
                           ("attn.wv", "self_attn.v_proj.weight"), ("attn.wo", "self_attn.o_proj.weight"),
                           ("ff.w1", "mlp.gate_proj.weight"), ("ff.w3", "mlp.up_proj.weight"),
                           ("ff.w2", "mlp.down_proj.weight"), ("norm_a", "input_layernorm.weight"),
                           ("norm_f", "post_attention_layernorm.weight")):
            m[b + llama] = w[a + toy]
    x = P.embed(m["model.embed_tokens.weight"], torch.tensor(ids))
    pos = torch.arange(len(ids))
    kvs = []
    for i in range(c.depth):
        x, kv = P.decoder_block(x, pos, cfg, m, i, window=c.window if i % 2 else None)
        kvs.append(kv)
    x, _ = P.decoder_block(x, pos, cfg, m, 1, window=c.window, shared_kv=kvs[1])
    return P.linear(P.rms_norm(x, m["model.norm.weight"], c.eps), m["model.embed_tokens.weight"])


def read_folder(d):
    return P.read_model_dir(d)     # through the `safetensors` package, which the product path does not use


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_toy_architecture_from_folder_to_tokens(tmp_path, dtype):
    import janus_b200
    from janus_b200.config import ConfigError, registered_architectures
    from janus_b200.engine import StepEntry
    from janus_b200.weights import write_random_model
    register()
    assert NAME in registered_architectures()
    d = write_random_model(TOY, str(tmp_path / "toy"), seed=21, dtype=dtype, norm_std=0.02)
    cfg, w = read_folder(d)
    assert cfg["architectures"] == [NAME] and "width" in cfg and "hidden_size" not in cfg
    assert "blocks.2.ff.w3" in w and "tokens.table" in w and len(w) == 2 + 9 * 3
    c = ToyConfig.from_dict({k: v for k, v in cfg.items()})
    model = janus_b200.load(d, dtype=dtype, max_tokens=1024, max_slots=4)
    assert type(model.config) is ToyConfig
    # two cache groups (all keys; a window of 40), and the place that runs layer 1 again holds no cache of its own
    groups = model.engine.cache.groups
    assert sorted(g.spec.window for g in groups) == [0, 40]
    # the step function: prompts of unequal lengths in one step, cut, then one token each, past the window's edge
    seqs = [random_tokens(n, c.vocab, 40 + n) for n in (90, 23)]
    ref = [plain_toy(c, w, ids) for ids in seqs]
    tol = tol_for(dtype)
    a, b = model.alloc_slot(), model.alloc_slot()
    first = model.step([StepEntry(a, seqs[0][:50], range(50)), StepEntry(b, seqs[1][:10], range(10))]).cpu()
    assert rel_err(first[:50], ref[0][:50]) < tol and rel_err(first[50:], ref[1][:10]) < tol
    for j in range(40):
        entries = [StepEntry(a, [seqs[0][50 + j]], [0])]
        if 10 + j < len(seqs[1]):
            entries.append(StepEntry(b, [seqs[1][10 + j]], [0]))
        out = model.step(entries).cpu()
        assert rel_err(out[0:1], ref[0][50 + j:51 + j]) < tol, f"position {50 + j}"
        if len(entries) == 2:
            assert rel_err(out[1:2], ref[1][10 + j:11 + j]) < tol
    model.free_slot(a)
    model.free_slot(b)
    # generation through the entry point: greedy tokens are the plain argmax given the tokens before; the toy's
    # own stop token (its configuration's `end_tokens`) ends a sequence and is not part of the output
    prompts = [random_tokens(n, c.vocab - 1, 5 + n) for n in (7, 30, 3)]
    out, reasons, stats = model.generate(prompts, max_tokens=12, return_reasons=True, batch_size=2)
    assert stats.batches == 2
    for p, o, r in zip(prompts, out, reasons):
        logits = plain_toy(c, w, list(p) + list(o) + [0])
        for j, tok in enumerate(o):
            row = logits[len(p) - 1 + j]
            if dtype == "float32":
                assert tok == P.argmax_lowest(row)
            else:
                assert float(row.max() - row[tok]) <= BF16_TOL * float(row.abs().max())
        assert 310 not in o and (r == "length" and len(o) == 12 or r == "stop")
    # what does not fit is said in the toy's own words
    with pytest.raises(ConfigError, match="groups"):
        ToyConfig.from_dict(dict(TOY, groups=4))
    model.engine.cache.check()


def test_the_replay_program_serves_an_architecture_that_a_plugin_module_registers(tmp_path):
    """`JANUS_PLUGINS` names modules to import before an architecture is looked up: `bin/trace_run`, a process
    of its own, replays the toy architecture's folder (a prompt, then tokens one by one) with this file as the
    plugin, and its logits match the plain parts."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np
    from helpers import ROOT
    from janus_b200.weights import write_random_model
    register()
    d = write_random_model(TOY, str(tmp_path / "toy"), seed=22, dtype="float32", norm_std=0.02)
    (tmp_path / "toy_plugin.py").write_text("import test_toy_architecture\ntest_toy_architecture.register()\n")
    cfg, w = read_folder(d)
    c = ToyConfig.from_dict(cfg)
    ids = random_tokens(60, c.vocab, 3)
    steps = [dict(step=0, entries=[dict(id="a", tokens=ids[:50], want=[0, 49])], end=[])]
    steps += [dict(step=j + 1, entries=[dict(id="a", tokens=[ids[50 + j]], want=[0])], end=["a"] if j == 9 else [])
              for j in range(10)]
    env = dict(os.environ, JANUS_PLUGINS="toy_plugin",
               PYTHONPATH=os.pathsep.join([str(tmp_path), os.path.join(ROOT, "tests"), os.environ.get("PYTHONPATH", "")]))
    out = tmp_path / "out"
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", "float32",
                          "--out", str(out), "--max-tokens", "128"],
                         input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
                         timeout=600, env=env)
    assert res.returncode == 0, res.stderr[-2000:]
    ref = plain_toy(c, w, ids).numpy()
    got = np.concatenate([np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, c.vocab) for s in steps])
    assert rel_err(torch.from_numpy(got), torch.from_numpy(ref[[0] + list(range(49, 60))])) < tol_for("float32")
