"""safetensors reading and writing, weight errors, random-weights mode."""
import json
import os
import struct

import pytest
import torch

from helpers import TINY_A, TINY_B
from janus_b200.config import LlamaConfig, resolve_architecture
from janus_b200.weights import (FolderCheckpoint, RandomCheckpoint, SafetensorsError, SafetensorsFile,
                                TensorSpec, WeightError, check_names, load_named, save_file,
                                write_random_model)


def test_round_trip_against_the_safetensors_package(tmp_path):
    from safetensors.torch import load_file, save_file as st_save
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int64).view(2, 3)}
    ours = str(tmp_path / "ours.safetensors")
    save_file(t, ours)
    theirs = load_file(ours)                      # their reader, our writer
    for k in t:
        assert torch.equal(theirs[k], t[k])
    st_save(t, str(tmp_path / "theirs.safetensors"))
    f = SafetensorsFile(str(tmp_path / "theirs.safetensors"))   # our reader, their writer
    assert sorted(f.names()) == ["a", "b", "c"]
    for k in t:
        assert torch.equal(f.tensor(k), t[k]) and f.shape(k) == tuple(t[k].shape)


def test_corrupt_files(tmp_path):
    p = tmp_path / "x.safetensors"
    p.write_bytes(b"abc")
    with pytest.raises(SafetensorsError, match="too small"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 10_000) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 5) + b"{bad}")
    with pytest.raises(SafetensorsError, match="JSON"):
        SafetensorsFile(str(p))
    save_file({"w": torch.zeros(4, 4)}, str(p))
    data = p.read_bytes()
    p.write_bytes(data[:-8])                       # truncated
    with pytest.raises(SafetensorsError, match="outside"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4, 4], "data_offsets": [0, 60]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + bytes(64))
    with pytest.raises(SafetensorsError, match="needs 64 bytes"):
        SafetensorsFile(str(p))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    arch = resolve_architecture(TINY_A)
    specs = arch.weight_specs(LlamaConfig.from_dict(TINY_A))
    ck = RandomCheckpoint(specs, seed=3, dtype="float32")
    tensors = {n: ck.tensor(n) for n in ck.names()}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 32)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    save_file(tensors, str(tmp_path / "model.safetensors"))
    with pytest.raises(WeightError) as e:
        load_named(FolderCheckpoint(str(tmp_path)), specs)
    msg = str(e.value)
    assert "model.layers.1.mlp.up_proj.weight" in msg and "model.norm.weight" in msg      # missing
    assert "rotary_emb.inv_freq" in msg                                                     # unexpected
    assert "q_proj.weight: expected [64, 64], got [64, 32]" in msg                          # wrong shape
    assert "missing tensors (2)" in msg and "unexpected tensors (1)" in msg and "wrong shapes (1)" in msg


def test_missing_folder_contents(tmp_path):
    with pytest.raises(WeightError, match="no weights"):
        FolderCheckpoint(str(tmp_path))


def test_tied_head_needs_no_lm_head_and_untied_does():
    b = resolve_architecture(TINY_B)
    names = [s.name for s in b.weight_specs(LlamaConfig.from_dict(TINY_B))]
    assert "lm_head.weight" not in names
    a = resolve_architecture(TINY_A)
    specs = a.weight_specs(LlamaConfig.from_dict(TINY_A))
    assert "lm_head.weight" in [s.name for s in specs]
    ck = RandomCheckpoint([s for s in specs if s.name != "lm_head.weight"], seed=0)
    with pytest.raises(WeightError, match="lm_head.weight"):
        check_names(ck, specs)


def test_kept_dtypes(tmp_path):
    save_file({"m": torch.randn(4, 4).to(torch.float16), "n": torch.ones(4), "t": torch.arange(4, dtype=torch.int64)},
              str(tmp_path / "model.safetensors"))
    specs = [TensorSpec("m", (4, 4)), TensorSpec("n", (4,)), TensorSpec("t", (4,))]
    named = load_named(FolderCheckpoint(str(tmp_path)), specs)
    assert named["m"].dtype == torch.bfloat16      # 16-bit floats are kept in bfloat16
    assert named["n"].dtype == torch.float32       # stored in 32-bit stays so
    assert named["t"].dtype == torch.int32         # integer tables as int32
    # the float32 engine widens a float16 tensor exactly: no rounding to bfloat16 on the way
    wide = load_named(FolderCheckpoint(str(tmp_path)), specs, engine_dtype=torch.float32)
    stored = FolderCheckpoint(str(tmp_path)).tensor("m")
    assert stored.dtype == torch.float16 and wide["m"].dtype == torch.float32
    assert torch.equal(wide["m"], stored.float())
    assert not torch.equal(named["m"].float(), stored.float())
    assert wide["t"].dtype == torch.int32


@pytest.mark.parametrize("cfg, dtype", [(TINY_A, "float32"), (TINY_B, "bfloat16")])
def test_random_model_folder(tmp_path, cfg, dtype):
    d = write_random_model(cfg, str(tmp_path / "m"), seed=5, dtype=dtype)
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    arch = resolve_architecture(json.load(open(os.path.join(d, "config.json"))))
    config = arch.config_class.from_dict(json.load(open(os.path.join(d, "config.json"))))
    assert config == arch.config_class.from_dict(dict(cfg, torch_dtype=dtype))
    ck = FolderCheckpoint(d)
    check_names(ck, arch.weight_specs(config))
    want = torch.float32 if dtype == "float32" else torch.bfloat16
    assert all(ck.dtype(n) == want for n in ck.names())
    w = ck.tensor("model.layers.0.mlp.down_proj.weight").float()
    assert abs(float(w.std()) - 0.02) < 0.004
    g = ck.tensor("model.norm.weight").float()
    assert abs(float(g.mean()) - 1.0) < 0.02 and float(g.std()) > 0.0
    # the same seed gives the same folder, another seed another one
    d2 = write_random_model(cfg, str(tmp_path / "m2"), seed=5, dtype=dtype)
    d3 = write_random_model(cfg, str(tmp_path / "m3"), seed=6, dtype=dtype)
    a, b2, c3 = (open(os.path.join(x, "model.safetensors"), "rb").read() for x in (d, d2, d3))
    assert a == b2 and a != c3


def test_random_tensor_does_not_depend_on_other_tensors():
    s1 = [TensorSpec("x", (8, 8)), TensorSpec("y", (4,), "ones")]
    s2 = [TensorSpec("y", (4,), "ones"), TensorSpec("z", (2, 2)), TensorSpec("x", (8, 8))]
    a, b = RandomCheckpoint(s1, 7, "float32"), RandomCheckpoint(s2, 7, "float32")
    assert torch.equal(a.tensor("x"), b.tensor("x")) and torch.equal(a.tensor("y"), b.tensor("y"))


def test_sharded_folder(tmp_path):
    """Shards named by model.safetensors.index.json read as one checkpoint; a shard that is missing, an
    index that is none and a tensor stored twice are weight errors."""
    from helpers import make_model_dir
    arch = resolve_architecture(TINY_B)
    specs = arch.weight_specs(LlamaConfig.from_dict(TINY_B))
    one = make_model_dir(TINY_B, str(tmp_path / "one"), seed=4, dtype="bfloat16")
    three = make_model_dir(TINY_B, str(tmp_path / "three"), seed=4, dtype="bfloat16", shards=3)
    files = sorted(os.listdir(three))
    assert "model.safetensors" not in files and len([f for f in files if f.endswith(".safetensors")]) == 3
    a, b = FolderCheckpoint(one), FolderCheckpoint(three)
    check_names(b, specs)
    assert sorted(a.names()) == sorted(b.names())
    for n in a.names():
        assert torch.equal(a.tensor(n), b.tensor(n)) and a.shape(n) == b.shape(n) and a.dtype(n) == b.dtype(n)
    # a tensor that two shards store
    twice = os.path.join(three, files[1])
    dup = SafetensorsFile(os.path.join(three, files[2]))
    name = dup.names()[0]
    extra = SafetensorsFile(twice)
    save_file(dict({n: extra.tensor(n).clone() for n in extra.names()}, **{name: dup.tensor(name).clone()}),
              str(tmp_path / "dup.safetensors"))
    del extra, dup
    os.replace(str(tmp_path / "dup.safetensors"), twice)
    with pytest.raises(WeightError, match="stored twice"):
        FolderCheckpoint(three)
    # a shard that is not there
    os.remove(twice)
    with pytest.raises(WeightError, match="cannot open"):
        FolderCheckpoint(three)
    # an index that is none
    with open(os.path.join(three, "model.safetensors.index.json"), "w") as f:
        f.write('{"metadata": {}}')
    with pytest.raises(WeightError, match="no shard index"):
        FolderCheckpoint(three)


def test_random_values_are_a_function_of_seed_name_and_index():
    """The generator against its definition in plain integers: element i is the sum of twelve 16-bit pieces of
    three splitmix64 values of key + (3 i + d + 1) * golden, centred and scaled by 2^-16.  Chunks and the order
    of creation change nothing."""
    from janus_b200.weights.random_init import standard_normal, tensor_key
    M = (1 << 64) - 1

    def mix(x):
        x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & M
        x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & M
        return x ^ (x >> 31)

    def element(key, i):
        total = 0
        for d in range(3):
            h = mix((key + (3 * i + d + 1) * 0x9E3779B97F4A7C15) & M)
            total += sum((h >> s) & 0xFFFF for s in (0, 16, 32, 48))
        return (total - 6 * 65535) / 65536.0

    key = tensor_key(7, "model.layers.0.mlp.up_proj.weight")
    assert key == tensor_key(7, "model.layers.0.mlp.up_proj.weight") != tensor_key(8, "model.layers.0.mlp.up_proj.weight")
    z = standard_normal(key, 0, 1000, "cpu")
    assert z.dtype == torch.float32
    for i in (0, 1, 2, 499, 999):
        assert float(z[i]) == element(key, i)
    assert torch.equal(standard_normal(key, 990, 10, "cpu"), z[990:])
    big = standard_normal(key, 0, 1 << 18, "cpu")
    assert abs(float(big.mean())) < 0.01 and abs(float(big.std()) - 1.0) < 0.01
    ck = RandomCheckpoint([TensorSpec("model.layers.0.mlp.up_proj.weight", (20, 50))], 7, "float32", std=0.5)
    assert torch.equal(ck.tensor("model.layers.0.mlp.up_proj.weight").view(-1), z * 0.5)
