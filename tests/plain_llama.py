"""Plain, slow Llama decoder written from the formulas of DaCodeChick/Janus.

This file is the oracle of the test-suite.  It recomputes whole sequences with
no cache, one function per part, in float32 (or float64) on the CPU, and shares
no code with ``janus_b200``.  The reference project is Rust + WGSL shaders that
run through a graphics API and cannot be built or run here (no cargo, no
rustc, no graphics stack), so this file rests on the reference's formulas,
cited as ``file:line`` inside ``crates/janus-engine`` (abbreviated ``JE/``).

Where the reference has no formula (explicit ``head_dim``, ``rope_theta``,
llama3 frequency scaling, tied head, per-sequence positions) the config.json
key's usual meaning is used and said so in the docstring.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch

Tensor = torch.Tensor


# --------------------------------------------------------------------------
# model folder
# --------------------------------------------------------------------------
def read_model_dir(model_dir: str, dtype=torch.float32):
    """Return (config dict, {name: tensor as `dtype`}) of a model folder.

    The folder layout is the reference's directory mode: ``config.json`` beside
    ``model.safetensors`` (JE/examples/inference.rs:118-125).  Reading goes
    through the `safetensors` package, which the product path does not use.
    """
    from safetensors import safe_open

    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    tensors = {}
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.exists(single):
        files = [single]
    else:      # a sharded folder: every file that model.safetensors.index.json names
        with open(os.path.join(model_dir, "model.safetensors.index.json")) as f:
            files = sorted({os.path.join(model_dir, v) for v in json.load(f)["weight_map"].values()})
    for path in files:
        with safe_open(path, framework="pt") as f:
            for name in f.keys():
                tensors[name] = f.get_tensor(name).to(dtype)
    return cfg, tensors


def cfg_get(cfg: dict, key: str):
    """config.json keys with the defaults of JE/src/model/config.rs:61-98,235-271."""
    if key == "num_key_value_heads":
        v = cfg.get(key)
        return cfg["num_attention_heads"] if v is None else v          # config.rs:235-241
    if key == "head_dim":
        v = cfg.get(key)
        return cfg["hidden_size"] // cfg["num_attention_heads"] if v is None else v  # config.rs:246-248
    if key == "intermediate_size":
        v = cfg.get(key)
        return 4 * cfg["hidden_size"] if v is None else v               # config.rs:254-260
    if key == "rms_norm_eps":
        return cfg.get(key, 1e-5)                                       # config.rs:88-98
    if key == "rope_theta":
        return cfg.get(key, 10000.0)                                    # config.rs:299
    if key == "tie_word_embeddings":
        return bool(cfg.get(key, False))
    return cfg[key]


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------
def embed(table: Tensor, ids: Tensor) -> Tensor:
    """x[t, :] = table[ids[t], :], no scaling (JE/src/compute/shaders/embed.wgsl:46-62)."""
    return table[ids.long()]


def rms_norm(x: Tensor, gamma: Tensor, eps: float) -> Tensor:
    """y = x / sqrt(mean(x^2) + eps) * gamma.

    JE/src/compute/shaders/activations.wgsl:81-133: sum of squares, divide by
    the width, add eps, sqrt, then divide and multiply by gamma (no +1 offset).
    """
    ms = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    rms = torch.sqrt(ms + eps)
    return (x / rms) * gamma


def rope_inv_freq(head_dim: int, theta: float, scaling: Optional[dict]) -> Tensor:
    """Inverse rotary frequencies 1 / theta^(2i/head_dim), i in [0, head_dim/2).

    JE/src/model/transformer/constructor.rs:467-475 computes
    ``theta_base.powf(2*i/head_dim)`` in f32 and divides the position by it.
    ``rope_scaling`` of type "llama3" (not in the reference; config.json's
    meaning): per frequency, with wavelength lambda = 2*pi/inv_freq, keep it if
    lambda < orig/high_freq_factor, divide by `factor` if lambda >
    orig/low_freq_factor, else blend linearly in orig/lambda between the two.
    All in float32.
    """
    half = head_dim // 2
    i = torch.arange(half, dtype=torch.float32)
    exponent = (2.0 * i) / float(head_dim)
    th = torch.pow(torch.tensor(float(theta), dtype=torch.float32), exponent)
    inv = 1.0 / th
    if scaling is None:
        return inv
    kind = scaling.get("rope_type", scaling.get("type"))
    if kind in (None, "default"):
        return inv
    if kind != "llama3":
        raise ValueError(f"plain implementation knows no rope scaling '{kind}'")
    factor = float(scaling["factor"])
    low = float(scaling["low_freq_factor"])
    high = float(scaling["high_freq_factor"])
    orig = float(scaling["original_max_position_embeddings"])
    out = torch.empty_like(inv)
    for j in range(half):
        f = float(inv[j])
        wavelen = 2.0 * math.pi / f
        if wavelen < orig / high:
            out[j] = f
        elif wavelen > orig / low:
            out[j] = f / factor
        else:
            smooth = (orig / wavelen - low) / (high - low)
            out[j] = (1.0 - smooth) * f / factor + smooth * f
    return out.to(torch.float32)


def rope_cos_sin(positions: Tensor, inv_freq: Tensor):
    """angle = position * inv_freq in f32; cos and sin in f32
    (JE/src/model/transformer/constructor.rs:475-479)."""
    ang = positions.to(torch.float32)[:, None] * inv_freq[None, :].to(torch.float32)
    return torch.cos(ang), torch.sin(ang)


def apply_rope(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    """Half-split rotation of the pairs (i, i + head_dim/2).

    x: [T, heads, head_dim]; cos, sin: [T, head_dim/2].
    y_i = x_i cos - x_{i+h} sin ; y_{i+h} = x_i sin + x_{i+h} cos
    (JE/src/compute/shaders/rope.wgsl:55-76).
    """
    half = x.shape[-1] // 2
    x0, x1 = x[..., :half], x[..., half:]
    c, s = cos[:, None, :].to(x.dtype), sin[:, None, :].to(x.dtype)
    return torch.cat([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1)


def attention(q: Tensor, k: Tensor, v: Tensor, window: Optional[int] = None) -> Tensor:
    """Causal grouped-query attention over a whole sequence.

    q: [T, nh, hd], k, v: [T, nkv, hd] (k already rotated).  For query head h
    the key/value head is floor(h*nkv/nh) (JE/src/compute/shaders/attention.wgsl:96,167);
    score = (q . k) * (1/sqrt(hd)), the scale applied after the dot
    (attention.wgsl:108-115, JE/src/compute/ops/attention.rs:98); keys t <= own
    position only (attention.wgsl:77); softmax = exp(s - max) / sum
    (JE/src/compute/shaders/softmax.wgsl:29-50); out = sum_t p_t v_t
    (attention.wgsl:170-185).  `window` (not in the reference) keeps only the
    last `window` keys, the query's own position included.
    """
    T, nh, hd = q.shape
    nkv = k.shape[1]
    scale = 1.0 / math.sqrt(hd)
    out = torch.empty_like(q)
    pos = torch.arange(T)
    allowed = pos[None, :] <= pos[:, None]
    if window is not None:
        allowed &= pos[None, :] > (pos[:, None] - window)
    for h in range(nh):
        kvh = (h * nkv) // nh
        s = (q[:, h, :] @ k[:, kvh, :].T) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        e = torch.exp(s - m)
        p = e / e.sum(dim=-1, keepdim=True)
        out[:, h, :] = p @ v[:, kvh, :]
    return out


def linear(x: Tensor, w: Tensor) -> Tensor:
    """y = x W^T with W stored [out, in], no bias
    (JE/src/compute/shaders/gemm.wgsl:1-13,99-139)."""
    return x @ w.T


def silu(x: Tensor) -> Tensor:
    """x * 1/(1+exp(-x)) (JE/src/compute/shaders/activations.wgsl:20-35)."""
    return x * (1.0 / (1.0 + torch.exp(-x)))


def swiglu_ffn(x: Tensor, w_gate: Tensor, w_up: Tensor, w_down: Tensor) -> Tensor:
    """down( silu(gate(x)) * up(x) ) (JE/src/model/block.rs:383-444)."""
    return linear(silu(linear(x, w_gate)) * linear(x, w_up), w_down)


def attention_block(x: Tensor, positions: Tensor, cfg: dict, w: Dict[str, Tensor], layer: int,
                    window: Optional[int] = None, shared_kv=None):
    """q/k/v projections, rope on q and k, attention, o projection
    (JE/src/model/block.rs:239-352).  Returns (out, (k_rot, v)) so that another
    layer of a schedule can read this layer's keys and values."""
    nh = cfg_get(cfg, "num_attention_heads")
    nkv = cfg_get(cfg, "num_key_value_heads")
    hd = cfg_get(cfg, "head_dim")
    p = f"model.layers.{layer}.self_attn."
    T = x.shape[0]
    inv = rope_inv_freq(hd, cfg_get(cfg, "rope_theta"), cfg.get("rope_scaling"))
    cos, sin = rope_cos_sin(positions, inv)
    q = linear(x, w[p + "q_proj.weight"]).view(T, nh, hd)
    q = apply_rope(q, cos, sin)
    if shared_kv is None:
        k = linear(x, w[p + "k_proj.weight"]).view(T, nkv, hd)
        v = linear(x, w[p + "v_proj.weight"]).view(T, nkv, hd)
        k = apply_rope(k, cos, sin)
    else:
        k, v = shared_kv
    o = attention(q, k, v, window=window).reshape(T, nh * hd)
    return linear(o, w[p + "o_proj.weight"]), (k, v)


def decoder_block(x: Tensor, positions: Tensor, cfg: dict, w: Dict[str, Tensor], layer: int,
                  window: Optional[int] = None, shared_kv=None):
    """Pre-norm block: h1 = x + attn(norm(x)); out = h1 + ffn(norm(h1))
    (JE/src/model/block.rs:223-233,355-363,370-380,447-455)."""
    eps = cfg_get(cfg, "rms_norm_eps")
    p = f"model.layers.{layer}."
    a, kv = attention_block(rms_norm(x, w[p + "input_layernorm.weight"], eps), positions, cfg, w,
                            layer, window=window, shared_kv=shared_kv)
    h1 = x + a
    n = rms_norm(h1, w[p + "post_attention_layernorm.weight"], eps)
    f = swiglu_ffn(n, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                   w[p + "mlp.down_proj.weight"])
    return h1 + f, kv


def lm_head_weight(cfg: dict, w: Dict[str, Tensor]) -> Tensor:
    """`lm_head.weight`, or the embedding table when the head is tied or the
    tensor is absent (the reference requires it, JE/examples/inference.rs:291;
    tying is config.json's `tie_word_embeddings`)."""
    if cfg_get(cfg, "tie_word_embeddings") or "lm_head.weight" not in w:
        return w["model.embed_tokens.weight"]
    return w["lm_head.weight"]


def forward(cfg: dict, w: Dict[str, Tensor], ids: Sequence[int],
            schedule: Optional[List] = None, window: Optional[int] = None) -> Tensor:
    """Logits [T, vocab] of one whole sequence from position 0
    (JE/src/model/transformer/forward.rs:25-119: embed, blocks, final norm, head).

    `schedule` (not in the reference) lists which layer runs at each place; an
    entry is a layer index or a pair (layer, place whose keys/values it reads).
    """
    ids_t = torch.as_tensor(list(ids), dtype=torch.long)
    dtype = w["model.embed_tokens.weight"].dtype
    x = embed(w["model.embed_tokens.weight"], ids_t).to(dtype)
    positions = torch.arange(len(ids_t))
    if schedule is None:
        schedule = list(range(cfg["num_hidden_layers"]))
    kvs = []
    for entry in schedule:
        if isinstance(entry, (tuple, list)):
            layer, reads = entry
            x, kv = decoder_block(x, positions, cfg, w, layer, window=window, shared_kv=kvs[reads])
        else:
            x, kv = decoder_block(x, positions, cfg, w, entry, window=window)
        kvs.append(kv)
    z = rms_norm(x, w["model.norm.weight"], cfg_get(cfg, "rms_norm_eps"))
    return linear(z, lm_head_weight(cfg, w))


# --------------------------------------------------------------------------
# sampling (JE/src/model/sampler.rs)
# --------------------------------------------------------------------------
def argmax_lowest(logits: Tensor) -> int:
    """Greedy pick; the lowest index wins a tie, as the GPU scan with strict
    `>` does (JE/src/compute/shaders/argmax.wgsl:43-51)."""
    best, best_i = None, 0
    for i, v in enumerate(logits.tolist()):
        if best is None or v > best:
            best, best_i = v, i
    return best_i


def apply_repetition_penalty(logits: Tensor, context: Sequence[int], penalty: float) -> Tensor:
    """For each token of the context, once per occurrence: a positive logit is
    divided by the penalty, another multiplied (sampler.rs:599-613)."""
    out = logits.clone()
    for t in context:
        if 0 <= t < out.numel():
            out[t] = out[t] / penalty if out[t] > 0 else out[t] * penalty
    return out


def apply_top_k(logits: Tensor, k: int) -> Tensor:
    """Values below the k-th largest become -inf; ties with it stay
    (sampler.rs:653-673)."""
    if k == 0 or k >= logits.numel():
        return logits
    thr = torch.sort(logits, descending=True).values[k - 1]
    return torch.where(logits < thr, torch.full_like(logits, float("-inf")), logits)


def softmax_probs(logits: Tensor) -> Tensor:
    """exp(x - max) / sum, non-finite entries count as 0 (sampler.rs:726-747)."""
    m = logits.max()
    e = torch.where(torch.isfinite(logits), torch.exp(logits - m), torch.zeros_like(logits))
    return e / e.sum()


def apply_top_p(probs: Tensor, p: float) -> Tensor:
    """Keep the smallest prefix of the descending order whose sum reaches p and
    renormalise (sampler.rs:683-717)."""
    order = torch.argsort(probs, descending=True, stable=True)
    csum = torch.cumsum(probs[order], dim=0)
    cutoff = int((csum >= p).nonzero()[0]) + 1 if bool((csum >= p).any()) else probs.numel()
    out = torch.zeros_like(probs)
    keep = order[:cutoff]
    out[keep] = probs[keep]
    return out / out.sum()


def sample_from_distribution(probs: Tensor, u: float) -> int:
    """First index whose running sum exceeds u; the last index otherwise
    (sampler.rs:756-772)."""
    c = 0.0
    for i, pr in enumerate(probs.tolist()):
        c += pr
        if u < c:
            return i
    return probs.numel() - 1


_M64 = (1 << 64) - 1


def uniform_for(seed: int, sequence: int, step: int) -> float:
    """Counter-based uniform in [0, 1) keyed by (seed, sequence, step).

    The reference draws from an unseeded thread RNG (sampler.rs:757-760); a
    keyed draw makes a sequence's tokens independent of what else is in the
    batch.  splitmix64 finaliser over the three keys, top 24 bits.
    """
    x = (seed * 0x9E3779B97F4A7C15 + sequence * 0xBF58476D1CE4E5B9 + step * 0x94D049BB133111EB
         + 0x2545F4914F6CDD1D) & _M64
    x ^= x >> 30
    x = (x * 0xBF58476D1CE4E5B9) & _M64
    x ^= x >> 27
    x = (x * 0x94D049BB133111EB) & _M64
    x ^= x >> 31
    return (x >> 40) / float(1 << 24)


def sampling_distribution(logits: Tensor, temperature: float, top_k: int = 0, top_p: float = 1.0,
                          repetition_penalty: float = 1.0, context: Sequence[int] = ()) -> Tensor:
    """Penalty, top-k, temperature, softmax, top-p in the reference's order
    (sampler.rs:196-197,622-646)."""
    x = logits.to(torch.float32)
    if repetition_penalty != 1.0:
        x = apply_repetition_penalty(x, context, repetition_penalty)
    if top_k > 0:
        x = apply_top_k(x, top_k)
    x = x / temperature
    probs = softmax_probs(x)
    if top_p < 1.0:
        probs = apply_top_p(probs, top_p)
    return probs


def sample(logits: Tensor, temperature: float, u: float, top_k: int = 0, top_p: float = 1.0,
           repetition_penalty: float = 1.0, context: Sequence[int] = ()) -> int:
    """temperature 0 means argmax (sampler.rs:200-206)."""
    if temperature == 0.0:
        x = logits.to(torch.float32)
        if repetition_penalty != 1.0:
            x = apply_repetition_penalty(x, context, repetition_penalty)
        return argmax_lowest(x)
    return sample_from_distribution(
        sampling_distribution(logits, temperature, top_k, top_p, repetition_penalty, context), u)


def generate(cfg: dict, w: Dict[str, Tensor], prompt: Sequence[int], max_new_tokens: int,
             temperature: float = 0.0, seed: int = 0, sequence: int = 0,
             stop_ids: Sequence[int] = (), top_k: int = 0, top_p: float = 1.0,
             repetition_penalty: float = 1.0) -> List[int]:
    """Whole-sequence recomputation per new token; the stop token is not
    appended (JE/src/model/transformer/generation.rs:241-263)."""
    ids = list(prompt)
    out: List[int] = []
    for step in range(max_new_tokens):
        logits = forward(cfg, w, ids)[-1]
        tok = sample(logits, temperature, uniform_for(seed, sequence, step), top_k, top_p,
                     repetition_penalty, out)
        if tok in stop_ids:
            break
        out.append(tok)
        ids.append(tok)
    return out
