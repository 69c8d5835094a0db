"""Configuration and registry (mirrors the reference's own config tests,
crates/janus-engine/src/model/config.rs:447-552 and tests/error_handling.rs)."""
import json

import pytest

from helpers import TINY_A, TINY_B
from janus_b200.config import (ConfigError, LlamaConfig, read_config_json, registered_architectures,
                               resolve_architecture)


def test_parse_tiny_configs():
    a = LlamaConfig.from_dict(TINY_A)
    assert (a.hidden_size, a.num_hidden_layers, a.num_attention_heads, a.num_key_value_heads) == (64, 2, 4, 2)
    assert a.head_dim == 16 and a.rope_scaling is None and a.eos_token_id == (250, 251)
    b = LlamaConfig.from_dict(TINY_B)
    assert b.head_dim == 40 and b.tie_word_embeddings and b.rms_norm_eps == 1e-6
    assert b.rope_scaling.factor == 4.0 and b.rope_scaling.original_max_position_embeddings == 32
    assert b.eos_token_id == (383,)


def test_defaults_follow_the_reference():
    c = LlamaConfig.from_dict(dict(hidden_size=128, num_hidden_layers=1, num_attention_heads=8, vocab_size=50))
    assert c.num_key_value_heads == 8           # config.rs:235-241
    assert c.head_dim == 16                      # config.rs:246-248
    assert c.intermediate_size == 512            # config.rs:254-260
    assert c.max_position_embeddings == 2048     # config.rs:265-271
    assert c.rms_norm_eps == 1e-5                # config.rs:96-98
    assert c.rope_theta == 10000.0               # config.rs:299
    assert c.architectures == ("LlamaForCausalLM",)


def test_round_trip_through_dict():
    for cfg in (TINY_A, TINY_B):
        c = LlamaConfig.from_dict(cfg)
        assert LlamaConfig.from_dict(json.loads(json.dumps(c.to_dict()))) == c


@pytest.mark.parametrize("patch, word", [
    (dict(hidden_size=None), "hidden_size"),
    (dict(vocab_size=0), "vocab_size"),
    (dict(num_attention_heads=5, head_dim=None), "divisible"),
    (dict(num_key_value_heads=3), "num_key_value_heads"),
    (dict(head_dim=15), "head_dim"),
    (dict(hidden_size=40000, head_dim=16), "hidden_size"),
    (dict(num_hidden_layers=300), "num_hidden_layers"),
    (dict(vocab_size=2_000_000), "vocab_size"),
    (dict(rms_norm_eps="tiny"), "rms_norm_eps"),
    (dict(rope_scaling=dict(rope_type="yarn", factor=2.0)), "rope_scaling"),
    (dict(rope_scaling=dict(rope_type="llama3", factor=2.0, low_freq_factor=4.0, high_freq_factor=1.0,
                            original_max_position_embeddings=32)), "low_freq_factor"),
    (dict(rope_scaling=dict(rope_type="llama3", factor=2.0)), "low_freq_factor"),
    (dict(eos_token_id=9999), "eos_token_id"),
    (dict(tie_word_embeddings="yes"), "tie_word_embeddings"),
])
def test_errors_name_the_key(patch, word):
    cfg = dict(TINY_A)
    for k, v in patch.items():
        if v is None:
            cfg.pop(k, None)
        else:
            cfg[k] = v
    with pytest.raises(ConfigError) as e:
        LlamaConfig.from_dict(cfg)
    assert word in str(e.value)


def test_registry_resolves_and_refuses():
    assert "LlamaForCausalLM" in registered_architectures()
    assert resolve_architecture(TINY_A).config_class is LlamaConfig
    assert resolve_architecture({k: v for k, v in TINY_A.items() if k != "architectures"}).name == "LlamaForCausalLM"
    with pytest.raises(ConfigError) as e:
        resolve_architecture(dict(TINY_A, architectures=["MambaForCausalLM"]))
    assert "MambaForCausalLM" in str(e.value) and "LlamaForCausalLM" in str(e.value)


def test_read_config_json_errors(tmp_path):
    with pytest.raises(ConfigError):
        read_config_json(str(tmp_path))                      # folder without config.json
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        read_config_json(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    assert read_config_json(str(tmp_path))["hidden_size"] == 96
    assert read_config_json(str(tmp_path / "config.json"))["hidden_size"] == 96


def test_a_width_the_bfloat16_products_cannot_take_is_refused_when_the_model_is_built():
    import torch
    from janus_b200.engine.model import DecoderModel
    from janus_b200.models.llama import llama_spec
    cfg = LlamaConfig.from_dict(dict(TINY_A, intermediate_size=100))      # rows of 200 bytes: no multiple of 16
    with pytest.raises(ValueError, match="multiple of 8"):
        DecoderModel(llama_spec(cfg), torch.bfloat16, torch.device("cpu"))
    DecoderModel(llama_spec(cfg), torch.float32, torch.device("cpu"))     # the 32-bit path has no such limit


def test_product_plan_picks_a_kernel_and_slices_that_the_kernels_take():
    """The cost estimate that picks a product's kernel and its slices of K: decode-sized products are cut so
    that two tiles per SM stream weights, few output tiles at prompt sizes are cut as well, large prompts run
    on CTA pairs, and nothing is cut that cannot add."""
    from janus_b200.kernels import ops
    for N, K in ((4096, 4096), (4096, 14336), (6144, 4096), (200, 120), (128, 64), (3072, 2048), (128256, 4096)):
        k_tiles = (K + 63) // 64
        for T in (1, 8, 64, 65, 128, 129, 200, 256, 511, 512, 1000, 2048, 8192):
            for mode in ("add", "store", "swiglu"):
                pair, split = ops.gemm_plan(T, N, K, mode)
                assert split >= 1 and (split == 1 or (mode == "add" and split <= max(1, k_tiles // 4)))
                assert not pair or T >= ops.GEMM_PAIR_MIN_TOKENS
                assert ops.gemm_plan(T, N, K, mode, allow_pairs=False)[0] is False
            assert ops.split_k_for(T, N, K) == ops.gemm_plan(T, N, K, "add")[1]
    assert ops.gemm_plan(8, 4096, 4096, "add") == (False, 13)      # 416 tiles in 3 waves of 5 steps each
    assert ops.gemm_plan(64, 4096, 4096, "add") == (False, 4)       # more tokens, more adds: one wave of 16 steps
    assert ops.gemm_plan(256, 4096, 4096, "add") == (False, 4)       # 32 output tiles: K in four slices
    assert ops.gemm_plan(512, 4096, 4096, "add") == (True, 2)        # 32 tiles of CTA pairs: K in two
    assert ops.gemm_plan(2048, 4096, 4096, "add") == (True, 1)        # 128 tiles on 74 pairs, but slices of 16 k-tiles are all epilogue
    # 128 tiles of 224 k-tiles on 74 pairs: a wave of whole tiles, then the other 54 in 4 slices each
    assert ops.gemm_plan_whole(2048, 4096, 14336, "add") == (True, 4, 74)
    assert ops.gemm_plan(2048, 14336, 4096, "swiglu") == (True, 1)
    assert ops.gemm_plan(64, 14336, 4096, "swiglu") == (False, 1)
    ops.set_deterministic(True)          # slices are summed in order: only the single-CTA kernel cuts K then
    try:
        for T in (1, 8, 64, 100, 256, 700, 2048):
            for N, K in ((4096, 4096), (4096, 14336), (6144, 4096)):
                pair, split = ops.gemm_plan(T, N, K, "add")
                assert not (pair and split > 1)
        assert ops.gemm_plan(8, 4096, 4096, "add") == (False, 4)      # one wave: a tile's ordered sum is not free
    finally:
        ops.set_deterministic(False)
    assert ops.gemm_plan(8, 4096, 4096, "add") == (False, 13)


def test_key_splits_of_decode_attention_stay_within_the_pages():
    """The split count of decode attention: at least one, never more splits than pages of the longest
    sequence allow, one split when the batch alone fills the SMs, and the measured picks at 8 kv heads."""
    from janus_b200.kernels import ops
    for n_seqs in (1, 2, 3, 8, 16, 37, 64, 100, 500):
        for nkv in (1, 2, 8, 40):
            for length in (1, 63, 64, 65, 2080, 4096, 32768, 131072):
                s = ops.decode_splits_for(n_seqs, nkv, length, 64)
                pages = (length + 63) // 64
                assert 1 <= s <= max(1, pages), (n_seqs, nkv, length, s)
    assert ops.decode_splits_for(8, 8, 4096, 64) == 4
    assert ops.decode_splits_for(64, 8, 4096, 64) == 1
    assert ops.decode_splits_for(1, 8, 4096, 64) == 16


def test_keys_the_kernels_cannot_honour_are_refused_by_name():
    """A config.json that asks for another activation or for biases is refused when it is read; it would
    otherwise run as if it had not asked."""
    from janus_b200.config import ConfigError, LlamaConfig
    from helpers import TINY_A
    assert LlamaConfig.from_dict(dict(TINY_A, hidden_act="silu", attention_bias=False, mlp_bias=False)).hidden_act == "silu"
    for key, value in (("hidden_act", "gelu"), ("attention_bias", True), ("mlp_bias", True)):
        with pytest.raises(ConfigError, match=key):
            LlamaConfig.from_dict(dict(TINY_A, **{key: value}))
    with pytest.raises(ConfigError, match="head_dim"):
        LlamaConfig.from_dict(dict(TINY_A, head_dim=272))
    # the keys survive a round trip through to_dict
    cfg = LlamaConfig.from_dict(TINY_A)
    assert LlamaConfig.from_dict(cfg.to_dict()) == cfg


def test_sizes_the_attention_kernels_cannot_take_are_refused_when_the_model_is_built():
    """head sizes and group sizes that a kernel would refuse at the first step are refused by the part's
    constructor: bfloat16 needs head_dim % 8 == 0 and at most 64 query heads per kv head unless the tensor-core
    prompt kernel takes the shape (groups up to 128); float32 takes them all up to head_dim 256."""
    import torch
    from janus_b200.config import resolve_architecture
    from helpers import TINY_A
    cpu = torch.device("cpu")

    def build(dtype, **over):
        cfg = dict(TINY_A, **over)
        arch = resolve_architecture(cfg)
        return arch.build(arch.config_class.from_dict(cfg), dtype, cpu)

    build(torch.float32, head_dim=12)
    with pytest.raises(ValueError, match="multiple of 8"):
        build(torch.bfloat16, head_dim=12)
    # 96 query heads on one kv head: the tensor-core prompt kernel takes groups of up to 128 at every head size
    # that the bfloat16 path has; 136 heads on one kv head are too many for it
    build(torch.bfloat16, hidden_size=96, num_attention_heads=96, num_key_value_heads=1, head_dim=136)
    build(torch.bfloat16, hidden_size=96, num_attention_heads=96, num_key_value_heads=1, head_dim=16)
    build(torch.float32, hidden_size=136, num_attention_heads=136, num_key_value_heads=1, head_dim=16)
    with pytest.raises(ValueError, match="query heads per key/value head"):
        build(torch.bfloat16, hidden_size=136, num_attention_heads=136, num_key_value_heads=1, head_dim=16)


def test_layers_share_one_rotary_table_no_longer_than_the_engine_needs():
    """Every layer names the same position encoding and gets the same object: one table on the device, not one
    per layer; its rows stop at the engine's longest sequence."""
    import torch
    from janus_b200.config import resolve_architecture
    from helpers import TINY_B
    cfg = dict(TINY_B, max_position_embeddings=131072)
    arch = resolve_architecture(cfg)
    model = arch.build(arch.config_class.from_dict(cfg), torch.float32, torch.device("cpu"))
    positions = [layer.mixer.position for layer in model.layers]
    assert len(positions) == 3 and all(p is positions[0] for p in positions)
    model.limit_positions(200)
    table = positions[0].fused_rotary_table()
    assert tuple(table.shape) == (200, 20, 2)
    assert all(layer.mixer.position.fused_rotary_table() is table for layer in model.layers)
    # another model with other constants gets a table of its own
    other_cfg = dict(cfg, rope_theta=10000.0)
    other = arch.build(arch.config_class.from_dict(other_cfg), torch.float32, torch.device("cpu"))
    assert other.layers[0].mixer.position is not positions[0]


def test_default_stop_tokens():
    """config.json's eos ids; for a Llama 3 vocabulary without any, the two ids the reference always stops at."""
    from janus_b200.config import LlamaConfig
    from helpers import TINY_A, TINY_B
    assert LlamaConfig.from_dict(TINY_A).stop_token_ids() == (250, 251)
    assert LlamaConfig.from_dict(TINY_B).stop_token_ids() == (383,)
    no_eos = {k: v for k, v in TINY_A.items() if k != "eos_token_id"}
    assert LlamaConfig.from_dict(no_eos).stop_token_ids() == ()
    assert LlamaConfig.from_dict(dict(no_eos, vocab_size=128256)).stop_token_ids() == (128001, 128009)
    assert LlamaConfig.from_dict(dict(TINY_A, vocab_size=128256)).stop_token_ids() == (250, 251)


def test_declared_argument_types_match_the_exported_c_functions():
    """`ops._SIGNATURES` names the argument types of every exported kernel function; a launch passes plain
    integers and floats, so a wrong letter would pass a pointer as an int.  Read the declarations from the
    sources and compare."""
    import re
    from pathlib import Path
    from janus_b200.kernels import ops
    csrc = Path(ops.__file__).resolve().parent.parent / "csrc"
    found = {}
    for path in csrc.glob("*.cu"):
        text = path.read_text()
        for m in re.finditer(r"JB_EXPORT\s+int\s+(\w+)\s*\(([^)]*)\)", text):
            name, args = m.group(1), m.group(2).strip()
            letters = ""
            for arg in [a.strip() for a in args.split(",") if a.strip()]:
                if "*" in arg or "cudaStream_t" in arg:
                    letters += "p"
                elif "unsigned long long" in arg:
                    letters += "u"
                elif "long long" in arg:
                    letters += "l"
                elif re.match(r"(const\s+)?float\b", arg):
                    letters += "f"
                elif re.match(r"(const\s+)?int\b", arg):
                    letters += "i"
                else:
                    raise AssertionError(f"{name}: unknown argument type in {arg!r}")
            found[name] = letters
    for name, signature in ops._SIGNATURES.items():
        assert found.get(name) == signature, f"{name}: declared {signature}, the source says {found.get(name)}"
    launched = {n for n, letters in found.items() if letters}      # everything but the head_dim queries
    assert launched - set(ops._SIGNATURES) <= {"jb_attention_bf16_decode_noalloc"}


def test_log_levels():
    from janus_b200 import log
    assert log.parse_level("debug") == 3 and log.parse_level("INFO") == 2 and log.parse_level(None) == 1
    assert log.parse_level("nonsense") == log.parse_level("warn")
    log.set_level("error")
    try:
        assert log.enabled("error") and not log.enabled("warn") and not log.enabled("debug")
    finally:
        log.set_level("warn")
    with log.nvtx_range("nothing happens without JANUS_NVTX=1"):
        pass


def test_a_second_gpu_in_one_process_is_refused_by_name():
    """The kernel libraries are set up for the device of their first launch: the first model binds the process to
    its GPU, a model on another one is refused when it is built."""
    import torch
    from janus_b200.kernels import ops
    saved = list(ops._bound_device)
    try:
        ops._bound_device.clear()
        ops.bind_device(torch.device("cuda:1"))
        ops.bind_device(torch.device("cuda:1"))
        with pytest.raises(ops.KernelError, match="cuda:1.*cuda:0|cuda:0.*process of its own"):
            ops.bind_device(torch.device("cuda:0"))
    finally:
        ops._bound_device[:] = saved


def test_the_reference_s_own_config_cases():
    """The JSON documents and expected values of the reference's config tests, read from its source as text
    (crates/janus-engine/src/model/config.rs:452-525): parsing, defaults, validation, head size."""
    parsed = LlamaConfig.from_dict(json.loads('''{"hidden_size": 4096, "num_hidden_layers": 32,
        "num_attention_heads": 32, "num_key_value_heads": 32, "vocab_size": 32000, "intermediate_size": 11008,
        "max_position_embeddings": 2048, "rms_norm_eps": 0.00001}'''))                     # config.rs:453-475
    assert (parsed.hidden_size, parsed.num_hidden_layers, parsed.num_attention_heads, parsed.vocab_size) == \
           (4096, 32, 32, 32000)
    assert parsed.head_dim == 128 and parsed.intermediate_size == 11008
    defaults = LlamaConfig.from_dict(json.loads('''{"hidden_size": 2048, "num_hidden_layers": 16,
        "num_attention_heads": 16, "vocab_size": 50000}'''))                                # config.rs:478-495
    assert defaults.num_key_value_heads == 16 and defaults.intermediate_size == 8192
    assert defaults.max_position_embeddings == 2048 and defaults.rms_norm_eps == 1e-5
    with pytest.raises(ConfigError, match="hidden_size"):                                   # config.rs:498-510
        LlamaConfig.from_dict(json.loads('''{"hidden_size": 0, "num_hidden_layers": 32,
            "num_attention_heads": 32, "vocab_size": 32000}'''))
    head = LlamaConfig.from_dict(json.loads('''{"hidden_size": 4096, "num_hidden_layers": 32,
        "num_attention_heads": 32, "vocab_size": 32000}'''))                                # config.rs:513-525
    assert head.head_dim == 128


def test_the_reference_s_own_error_handling_cases():
    """The JSON documents of the reference's error-handling tests, read from its source as text
    (crates/janus-engine/tests/error_handling.rs:9-177): each is refused or accepted as there, and a refusal
    names the keys that the reference's message names."""
    def refused(text, *words, resolve=False):
        cfg = json.loads(text)
        with pytest.raises((ConfigError, KeyError, ValueError)) as e:
            if resolve:
                resolve_architecture(cfg)
            else:
                LlamaConfig.from_dict(cfg)
        for w in words:
            assert w in str(e.value), (w, str(e.value))

    refused('{"hidden_size": 0, "num_hidden_layers": 32, "num_attention_heads": 32, "vocab_size": 32000}',
            "hidden_size")                                                                  # :9-26
    refused('{"hidden_size": 4097, "num_hidden_layers": 32, "num_attention_heads": 32, "vocab_size": 32000}',
            "hidden_size", "divisible", "num_attention_heads")                              # :29-47
    refused('{"hidden_size": 4096, "num_hidden_layers": 32, "num_attention_heads": 32, "num_key_value_heads": 5,'
            ' "vocab_size": 32000}', "num_attention_heads", "num_key_value_heads", "divisible")   # :50-69
    refused('{"architectures": ["GPT2LMHeadModel"], "hidden_size": 768, "num_hidden_layers": 12,'
            ' "num_attention_heads": 12, "vocab_size": 50257}', "GPT2LMHeadModel", "LlamaForCausalLM",
            resolve=True)                                                                   # :72-91
    refused('{"hidden_size": 100000, "num_hidden_layers": 32, "num_attention_heads": 32, "vocab_size": 32000}',
            "unreasonably large")                                                           # :94-110
    refused('{"num_hidden_layers": 32, "num_attention_heads": 32, "vocab_size": 32000}', "hidden_size")   # :164-177
    llama = json.loads('{"architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "num_hidden_layers": 32,'
                       ' "num_attention_heads": 32, "num_key_value_heads": 32, "vocab_size": 32000,'
                       ' "intermediate_size": 11008, "max_position_embeddings": 2048, "rms_norm_eps": 0.00001}')
    assert resolve_architecture(llama).config_class.from_dict(llama).num_hidden_layers == 32      # :113-132
    tiny = LlamaConfig.from_dict(json.loads(
        '{"architectures": ["LlamaForCausalLM"], "hidden_size": 2048, "num_hidden_layers": 22,'
        ' "num_attention_heads": 32, "num_key_value_heads": 4, "vocab_size": 32000, "intermediate_size": 5632,'
        ' "max_position_embeddings": 2048}'))                                               # :135-161
    assert (tiny.num_attention_heads, tiny.num_key_value_heads) == (32, 4)
