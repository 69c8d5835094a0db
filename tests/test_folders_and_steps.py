"""Model folders of other kinds and steps of other shapes than the replay tests bring: a folder stored in
float16, a folder in shards, random weights made on the device against the same made on the host, and a step
that mixes a chunk of one sequence's prompt with single tokens of others."""
import numpy as np
import pytest
import torch

import plain_llama as P
from helpers import TINY, make_model_dir, random_tokens, rel_err, tol_for

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_folder_stored_in_float16(tmp_path, dtype):
    """float16 on disk is widened exactly by the float32 engine (the plain implementation does the same) and
    rounded once to bfloat16 by the bfloat16 engine."""
    import janus_b200
    from janus_b200.engine import StepEntry
    from janus_b200.weights import FolderCheckpoint
    cfg = TINY["B"]
    d = make_model_dir(cfg, str(tmp_path / "m"), seed=21, dtype="float32", stored="float16")
    ck = FolderCheckpoint(d)
    assert all(ck.dtype(n) == torch.float16 for n in ck.names())
    pcfg, pw = P.read_model_dir(d)
    ids = random_tokens(90, cfg["vocab_size"], 3)
    ref = P.forward(pcfg, pw, ids).numpy()
    model = janus_b200.load(d, dtype=dtype, max_tokens=256)
    s = model.alloc_slot()
    rows = [model.step([StepEntry(s, ids[:70], range(70))]).cpu().numpy()]
    for j in range(70, 90):
        rows.append(model.step([StepEntry(s, [ids[j]], [0])]).cpu().numpy())
    model.check()
    assert rel_err(np.concatenate(rows), ref) < tol_for(dtype)


def test_a_folder_in_shards(tmp_path):
    import janus_b200
    from janus_b200.engine import StepEntry
    cfg = TINY["A"]
    d = make_model_dir(cfg, str(tmp_path / "m"), seed=22, dtype="float32", shards=4)
    pcfg, pw = P.read_model_dir(d)
    ids = random_tokens(50, cfg["vocab_size"], 4)
    model = janus_b200.load(d, dtype="float32", max_tokens=128)
    got = model.step([StepEntry(model.alloc_slot(), ids, range(50))]).cpu().numpy()
    assert rel_err(got, P.forward(pcfg, pw, ids).numpy()) < tol_for("float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_random_weights_have_the_same_bits_on_host_and_device(dtype):
    from janus_b200.weights import RandomCheckpoint, TensorSpec
    specs = [TensorSpec("a.weight", (131, 77)), TensorSpec("b.norm", (1000,), "ones"),
             TensorSpec("c.big", (4099, 4099))]            # c spans more than one chunk of the generator
    host = RandomCheckpoint(specs, 5, dtype, std=0.02, norm_std=0.02, device="cpu")
    dev = RandomCheckpoint(specs, 5, dtype, std=0.02, norm_std=0.02, device="cuda:0")
    for name in ("a.weight", "b.norm"):
        assert torch.equal(host.tensor(name), dev.tensor(name).cpu()), name
    big = dev.tensor("c.big").cpu().view(-1)
    n = big.numel()
    from janus_b200.weights.random_init import standard_normal, tensor_key
    for start in (0, (1 << 24) - 50, n - 100):           # the head, a chunk's seam, the tail
        z = standard_normal(tensor_key(5, "c.big"), start, 100, "cpu") * 0.02
        assert torch.equal(big[start:start + 100], z.to(big.dtype)), start


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_a_step_that_mixes_a_prompt_chunk_with_single_tokens(tmp_path, name, dtype):
    """Three sequences at different places: one brings the next 40 tokens of its prompt, two bring one token
    each.  The step runs them as one packed batch; every row matches the plain implementation."""
    import janus_b200
    from janus_b200.engine import StepEntry
    cfg = TINY[name]
    d = make_model_dir(cfg, str(tmp_path / "m"), seed=23, dtype=dtype)
    pcfg, pw = P.read_model_dir(d)
    V = cfg["vocab_size"]
    ids = [random_tokens(n, V, 31 + n) for n in (100, 30, 70)]
    ref = [P.forward(pcfg, pw, x).numpy() for x in ids]
    tol = tol_for(dtype)
    model = janus_b200.load(d, dtype=dtype, max_tokens=512)
    a, b, c = (model.alloc_slot() for _ in range(3))
    model.step([StepEntry(a, ids[0][:45], ()), StepEntry(b, ids[1][:12], ()), StepEntry(c, ids[2][:66], ())])
    # a continues its prompt across the page boundary at 64; b and c decode (c steps onto a new page next)
    out = model.step([StepEntry(b, [ids[1][12]], [0]), StepEntry(a, ids[0][45:85], range(40)),
                      StepEntry(c, [ids[2][66]], [0])]).cpu().numpy()
    assert rel_err(out[0:1], ref[1][12:13]) < tol
    assert rel_err(out[1:41], ref[0][45:85]) < tol
    assert rel_err(out[41:42], ref[2][66:67]) < tol
    # and the cache that this step left serves the next ones: all three decode together
    out = model.step([StepEntry(a, [ids[0][85]], [0]), StepEntry(b, [ids[1][13]], [0]),
                      StepEntry(c, [ids[2][67]], [0])]).cpu().numpy()
    assert rel_err(out[0:1], ref[0][85:86]) < tol and rel_err(out[1:2], ref[1][13:14]) < tol
    assert rel_err(out[2:3], ref[2][67:68]) < tol
    model.check()


def test_a_one_layer_model_decodes_many_steps_right():
    """With one layer only about ten kernels lie between the step that writes a cached row and the step that
    reads it, all launched with programmatic dependent launch; decode attention asks for cached pages before
    its dependency wait.  What orders the two steps is the copy of each step's index buffer at the step's
    start.  A hundred decode steps from a short prompt, across a page boundary, every row against plain."""
    import os
    import janus_b200
    from janus_b200.engine import StepEntry
    if os.environ.get("JANUS_PDL", "1") == "0":
        pytest.skip("this test is about programmatic dependent launch, which JANUS_PDL=0 turns off")
    cfg = dict(TINY["A"], num_hidden_layers=1)
    import tempfile
    with tempfile.TemporaryDirectory() as tmp:
        d = make_model_dir(cfg, os.path.join(tmp, "m"), seed=24, dtype="bfloat16")
        pcfg, pw = P.read_model_dir(d)
        model = janus_b200.load(d, dtype="bfloat16", max_tokens=256)
    ids = random_tokens(120, cfg["vocab_size"], 8)
    ref = P.forward(pcfg, pw, ids).numpy()
    s = model.alloc_slot()
    model.step([StepEntry(s, ids[:20], ())])
    rows = [model.step([StepEntry(s, [ids[j]], [0])]) for j in range(20, 120)]      # no host read in between
    got = torch.cat(rows).cpu().numpy()
    model.check()
    assert rel_err(got, ref[20:]) < tol_for("bfloat16")
