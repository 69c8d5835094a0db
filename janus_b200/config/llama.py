"""Typed configuration of the Llama dense decoder, read from config.json keys.

The reference reads `hidden_size, num_hidden_layers, num_attention_heads,
num_key_value_heads, vocab_size, intermediate_size, max_position_embeddings,
rms_norm_eps, architectures` (crates/janus-engine/src/model/config.rs:61-94) and
hard-codes the rest (rope base 10000, head_dim = hidden/heads, no tying:
config.rs:246-248,299).  Here the remaining config.json keys of the
architecture are read too: `head_dim, rope_theta, rope_scaling,
tie_word_embeddings, bos_token_id, eos_token_id, torch_dtype`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, KeyReader, read_config_json


@dataclass(frozen=True)
class RopeScaling:
    """`rope_scaling` of type "llama3": frequencies whose wavelength exceeds
    original_max/low_freq_factor are divided by `factor`, those shorter than
    original_max/high_freq_factor are kept, the band between is blended."""
    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    def to_dict(self) -> Dict[str, Any]:
        return {
            "rope_type": self.rope_type,
            "factor": self.factor,
            "low_freq_factor": self.low_freq_factor,
            "high_freq_factor": self.high_freq_factor,
            "original_max_position_embeddings": self.original_max_position_embeddings,
        }


def _parse_rope_scaling(raw: Any) -> Optional[RopeScaling]:
    if raw is None:
        return None
    if not isinstance(raw, dict):
        raise ConfigError(f"key 'rope_scaling' must be an object or null, got {raw!r}")
    kind = raw.get("rope_type", raw.get("type"))
    if kind in (None, "default"):
        return None
    if kind != "llama3":
        raise ConfigError(f"key 'rope_scaling.rope_type': unsupported value {kind!r} (supported: 'llama3', 'default')")
    r = KeyReader(raw)
    try:
        s = RopeScaling(
            rope_type="llama3",
            factor=r.number("factor"),
            low_freq_factor=r.number("low_freq_factor"),
            high_freq_factor=r.number("high_freq_factor"),
            original_max_position_embeddings=r.integer("original_max_position_embeddings"),
        )
    except ConfigError as e:
        raise ConfigError(f"in 'rope_scaling': {e}") from e
    if not s.low_freq_factor < s.high_freq_factor:
        raise ConfigError(
            f"key 'rope_scaling': low_freq_factor ({s.low_freq_factor}) must be below "
            f"high_freq_factor ({s.high_freq_factor})")
    return s


MAX_HEAD_DIM = 256                 # the attention kernels' largest head size, float32 and bfloat16
LLAMA3_VOCAB_SIZE = 128_256
LLAMA3_STOP_TOKEN_IDS = (128_001, 128_009)


@dataclass(frozen=True)
class LlamaConfig:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int = 2048
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_scaling: Optional[RopeScaling] = None
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    attention_bias: bool = False
    mlp_bias: bool = False
    bos_token_id: Optional[int] = None
    eos_token_id: Tuple[int, ...] = ()
    torch_dtype: Optional[str] = None
    architectures: Tuple[str, ...] = field(default_factory=lambda: ("LlamaForCausalLM",))

    ARCHITECTURE = "LlamaForCausalLM"

    # -- reading -----------------------------------------------------------
    @classmethod
    def from_dict(cls, data: Dict[str, Any]) -> "LlamaConfig":
        r = KeyReader(data)
        hidden = r.integer("hidden_size")
        heads = r.integer("num_attention_heads")
        kv_heads = r.integer("num_key_value_heads", default=heads)      # config.rs:235-241
        head_dim = r.integer("head_dim", default=None)
        if head_dim is None:
            if hidden % heads != 0:                                      # config.rs:161-170
                raise ConfigError(
                    f"key 'hidden_size' ({hidden}) must be divisible by 'num_attention_heads' "
                    f"({heads}) when 'head_dim' is not given")
            head_dim = hidden // heads                                   # config.rs:246-248
        archs = data.get("architectures")
        if archs is None:
            archs = (cls.ARCHITECTURE,)
        elif not (isinstance(archs, list) and all(isinstance(a, str) for a in archs)):
            raise ConfigError(f"key 'architectures' must be a list of strings, got {archs!r}")
        bos = r.integer("bos_token_id", default=None, minimum=0)
        cfg = cls(
            hidden_size=hidden,
            num_hidden_layers=r.integer("num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            intermediate_size=r.integer("intermediate_size", default=4 * hidden),   # config.rs:254-260
            vocab_size=r.integer("vocab_size"),
            max_position_embeddings=r.integer(
                "max_position_embeddings",
                default=r.integer("max_seq_length", default=2048)),     # config.rs:84-85,265-271
            rms_norm_eps=r.number("rms_norm_eps", default=1e-5),        # config.rs:88-98
            rope_theta=r.number("rope_theta", default=10000.0),         # config.rs:299
            rope_scaling=_parse_rope_scaling(data.get("rope_scaling")),
            tie_word_embeddings=r.boolean("tie_word_embeddings", default=False),
            hidden_act=r.string("hidden_act", default="silu"),
            attention_bias=r.boolean("attention_bias", default=False),
            mlp_bias=r.boolean("mlp_bias", default=False),
            bos_token_id=bos,
            eos_token_id=r.id_list("eos_token_id"),
            torch_dtype=r.string("torch_dtype", default=r.string("dtype", default=None)),
            architectures=tuple(archs),
        )
        cfg.validate()
        return cfg

    @classmethod
    def from_file(cls, path: str) -> "LlamaConfig":
        return cls.from_dict(read_config_json(path))

    # -- checks ------------------------------------------------------------
    def validate(self) -> None:
        """The reference's checks (config.rs:135-229) with `head_dim` free."""
        # sizes beyond reason first: what follows from them (a head size of 3125) would name the wrong key
        if self.hidden_size > 32768:                                     # config.rs:207-212
            raise ConfigError(f"key 'hidden_size' ({self.hidden_size}) is unreasonably large (>32768)")
        if self.num_hidden_layers > 256:                                 # config.rs:214-219
            raise ConfigError(f"key 'num_hidden_layers' ({self.num_hidden_layers}) is unreasonably large (>256)")
        if self.vocab_size > 1_000_000:                                  # config.rs:221-226
            raise ConfigError(f"key 'vocab_size' ({self.vocab_size}) is unreasonably large (>1M)")
        if self.num_attention_heads % self.num_key_value_heads != 0:     # config.rs:172-180
            raise ConfigError(
                f"key 'num_attention_heads' ({self.num_attention_heads}) must be divisible by "
                f"'num_key_value_heads' ({self.num_key_value_heads})")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"key 'head_dim' ({self.head_dim}) must be even for rotary positions")
        if self.head_dim > MAX_HEAD_DIM:
            raise ConfigError(f"key 'head_dim' ({self.head_dim}) is not supported: the attention kernels take "
                              f"head sizes up to {MAX_HEAD_DIM}")
        # The reference's block has one activation and no bias anywhere (SiLU:
        # compute/shaders/activations.wgsl:20-35; no bias is looked up: model/block.rs:239-276).
        # A config.json that asks for something else is refused, not run as if it had not asked.
        if self.hidden_act != "silu":
            raise ConfigError(f"key 'hidden_act' ({self.hidden_act!r}) is not supported: the feed-forward's "
                              f"gate is SiLU ('silu')")
        if self.attention_bias:
            raise ConfigError("key 'attention_bias' is true: attention projections with a bias are not supported")
        if self.mlp_bias:
            raise ConfigError("key 'mlp_bias' is true: feed-forward projections with a bias are not supported")
        for t in self.eos_token_id:
            if not 0 <= t < self.vocab_size:
                raise ConfigError(f"key 'eos_token_id': {t} is outside the vocabulary ({self.vocab_size})")

    def stop_token_ids(self) -> Tuple[int, ...]:
        """The tokens that end a sequence: config.json's `eos_token_id`; where it names none and the
        vocabulary is Llama 3's (128,256 entries), the two ids the reference always stops at,
        <|end_of_text|> 128001 and <|eot_id|> 128009
        (crates/janus-engine/src/model/transformer/generation.rs:6-7,241)."""
        if self.eos_token_id:
            return self.eos_token_id
        if self.vocab_size == LLAMA3_VOCAB_SIZE:
            return LLAMA3_STOP_TOKEN_IDS
        return ()

    # -- writing -----------------------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architectures": list(self.architectures),
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": None if self.rope_scaling is None else self.rope_scaling.to_dict(),
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
            "attention_bias": self.attention_bias,
            "mlp_bias": self.mlp_bias,
        }
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id) if len(self.eos_token_id) > 1 else self.eos_token_id[0]
        if self.torch_dtype is not None:
            d["torch_dtype"] = self.torch_dtype
        return d
