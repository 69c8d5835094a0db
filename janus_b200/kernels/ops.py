"""Python faces of the CUDA kernels: each function checks its tensors, passes
raw pointers and the current stream to the exported C function, and raises on
a non-zero return.  Nothing here computes; there is no other code path.
"""
from __future__ import annotations

import contextlib
import ctypes
import functools
import os
from typing import Optional, Tuple

import torch

from .build import library

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {dtype}")


_scope_stream = [None]


def _stream() -> int:
    s = _scope_stream[0]
    return s if s is not None else torch.cuda.current_stream().cuda_stream


@contextlib.contextmanager
def stream_scope():
    """Within the scope every launch goes to the stream that was current on entry: the question is asked
    once for a whole forward pass instead of once per kernel."""
    before = _scope_stream[0]
    _scope_stream[0] = torch.cuda.current_stream().cuda_stream
    try:
        yield
    finally:
        _scope_stream[0] = before


# Argument types of the exported C functions: p pointer, i int, l long long, u unsigned long long, f float;
# the last argument of every function is the stream.  Declared once per library, so that a launch passes
# plain Python integers and floats (a pointer is `tensor.data_ptr()`, None is a null pointer).
_SIGNATURES = {
    "jb_embed_gather": "pippiippp", "jb_rmsnorm": "pppifpiiiplp", "jb_residual_add": "ppilp",
    "jb_swiglu": "ppiiip", "jb_swiglu_f32_to_bf16": "piipiip", "jb_zero_f32": "plp",
    "jb_pack_weight_bf16": "piipp", "jb_rope_cache_write": "piipipppppiiiiiiip",
    "jb_gemm_f32": "pppiiiiiip", "jb_attention_f32": "pppppppiiiiiiifp",
    "jb_gemm_bf16": "pplipiiiiiiplpipp", "jb_gemm_bf16_pair": "pplipiiiiiiipp",
    "jb_gemm_bf16_pair_qkv_rope": "ppliippppppiiiipp",
    "jb_sample": "piipfiffppupppp",
    "jb_attention_bf16_prefill": "pppppppiiiiiiiifp", "jb_attention_bf16_decode": "ppppppppiiiiiiifip",
    "jb_attention_bf16_decode_fused": "pipppppppppiiiiiiifiip",
    "jb_attention_tc_prefill": "pppppppiiiiiiiiiifpp",
}
_CTYPES = {"p": ctypes.c_void_p, "i": ctypes.c_int, "l": ctypes.c_longlong, "u": ctypes.c_ulonglong,
           "f": ctypes.c_float}

_libs = {}


def _lib(stem: str, key=None, defines=None) -> ctypes.CDLL:
    """The built library `stem` (variant `key`, compiled with `defines(key)` or the dict `defines`);
    asked for on every launch, so the answer is remembered here."""
    lib = _libs.get((stem, key))
    if lib is None:
        lib = library(stem, defines(key) if callable(defines) else defines)
        for name, signature in _SIGNATURES.items():
            fn = getattr(lib, name, None)
            if fn is not None:
                fn.argtypes = [_CTYPES[c] for c in signature]
                fn.restype = ctypes.c_int
        _libs[(stem, key)] = lib
    return lib


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


# Whether the faces below check their tensors (device, contiguity, dtype, shape).  The engine turns the
# checks off for a step whose shape it has run before with the checks on: the same parts then hand the same
# kinds of tensors to the same kernels.
_checks = [True]


@contextlib.contextmanager
def unchecked():
    before = _checks[0]
    _checks[0] = False
    try:
        yield
    finally:
        _checks[0] = before


def _need(t: torch.Tensor, name: str, dtype=None, shape=None) -> None:
    if not _checks[0]:
        return
    if not t.is_cuda:
        raise KernelError(f"{name}: tensor must be on a CUDA device (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name}: tensor must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise KernelError(f"{name}: expected shape {tuple(shape)}, got {tuple(t.shape)}")


_launches = [0]


def launch_count() -> int:
    """Kernels of this library launched (or captured into a graph) so far."""
    return _launches[0]


_trace = [None]    # while a step is profiled: the list that takes (face, kernels, event after the launch)


@contextlib.contextmanager
def trace_launches():
    """Within the scope every launch of this library is followed by a CUDA event on the current stream; the
    list that is handed out holds (face, kernels, event), led by an event recorded on entry.  The time between
    two events is the time the stream spent on the launch between them (kernels run one after another on a
    stream; what overlaps under programmatic dependent launch is counted for the later kernel)."""
    before = _trace[0]
    start = torch.cuda.Event(enable_timing=True)
    start.record()
    events = [("start", 0, start)]
    _trace[0] = events
    try:
        yield events
    finally:
        _trace[0] = before


def _check(code: int, what: str, kernels: int = 1) -> None:
    if code == 0:
        _launches[0] += kernels
        if _trace[0] is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            _trace[0].append((what, kernels, ev))
        return
    if code >= 10000:
        names = {10001: "size not supported (see stderr)", 10002: "dtype not supported",
                 10003: "tensor map could not be encoded"}
        raise KernelError(f"{what}: {names.get(code, 'error')} (code {code})")
    raise KernelError(f"{what}: CUDA error {code}")


# -- embedding, norm, elementwise ---------------------------------------------
def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor,
                 feedback: Optional[torch.Tensor] = None, token_slot: Optional[torch.Tensor] = None) -> None:
    """out[t, :] = float32(table[ids[t], :]); a negative id stands for feedback[token_slot[t]]"""
    T, H = out.shape
    _need(table, "embed table")
    _need(ids, "token ids", torch.int32, (T,))
    _need(out, "embed out", torch.float32)
    if table.shape[1] != H:
        raise KernelError(f"embed: table width {table.shape[1]} != output width {H}")
    _check(_lib("elementwise").jb_embed_gather(
        _ptr(table), dtype_code(table.dtype), _ptr(ids), _ptr(out), T, H, _ptr(feedback), _ptr(token_slot),
        _stream()), "embed_gather")


def rmsnorm(x: torch.Tensor, gamma: torch.Tensor, eps: float, out: torch.Tensor,
            row_index: Optional[torch.Tensor] = None, clear: Optional[torch.Tensor] = None) -> None:
    """out[r] = x[row_index[r] or r] / sqrt(mean(x^2) + eps) * gamma.  `clear`: a float32
    scratch tensor (whole 16-byte vectors) that the same launch sets to zero."""
    rows, H = out.shape
    _need(x, "rmsnorm x", torch.float32)
    _need(gamma, "rmsnorm gamma", None, (H,))
    _need(out, "rmsnorm out")
    if x.shape[1] != H:
        raise KernelError(f"rmsnorm: input width {x.shape[1]} != output width {H}")
    if clear is not None:
        _need(clear, "rmsnorm clear", torch.float32)
    if row_index is not None:
        _need(row_index, "rmsnorm row_index", torch.int32, (rows,))
    elif x.shape[0] < rows:
        raise KernelError("rmsnorm: fewer input rows than output rows")
    _check(_lib("elementwise").jb_rmsnorm(
        _ptr(x), _ptr(row_index), _ptr(gamma), dtype_code(gamma.dtype), eps, _ptr(out),
        dtype_code(out.dtype), rows, H, _ptr(clear), 0 if clear is None else clear.numel(),
        _stream()), "rmsnorm")


def residual_add(residual: torch.Tensor, delta: torch.Tensor) -> None:
    """residual += float32(delta), elementwise, in place"""
    _need(residual, "residual", torch.float32)
    _need(delta, "delta", None, residual.shape)
    _check(_lib("elementwise").jb_residual_add(
        _ptr(residual), _ptr(delta), dtype_code(delta.dtype), residual.numel(), _stream()),
        "residual_add")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, c] = silu(gate_up[t, c]) * gate_up[t, I + c]"""
    T, I = out.shape
    _need(gate_up, "swiglu input", out.dtype, (T, 2 * I))
    _need(out, "swiglu out")
    _check(_lib("elementwise").jb_swiglu(_ptr(gate_up), _ptr(out), dtype_code(out.dtype), T, I, _stream()),
           "swiglu")


def swiglu_f32_to_bf16(gate_up: torch.Tensor, out: torch.Tensor, up_col: int) -> None:
    """out[t, c] = silu(gate_up[t, c]) * gate_up[t, up_col + c]; float32 in, bfloat16 out."""
    T, I = out.shape
    _need(gate_up, "swiglu input", torch.float32)
    _need(out, "swiglu out", torch.bfloat16)
    if gate_up.dim() != 2 or gate_up.shape[0] != T:
        raise KernelError(f"swiglu: input of shape {tuple(gate_up.shape)} does not hold {T} rows")
    _check(_lib("elementwise").jb_swiglu_f32_to_bf16(_ptr(gate_up), gate_up.shape[1], int(up_col), _ptr(out), T, I,
                                                      _stream()), "swiglu_f32_to_bf16")


def zero_f32(t: torch.Tensor) -> None:
    """Fill a float32 tensor with zeros (whole 16-byte vectors)."""
    _need(t, "zero target", torch.float32)
    _check(_lib("elementwise").jb_zero_f32(_ptr(t), t.numel(), _stream()), "zero_f32")


# -- rotary positions + cache append --------------------------------------------
def rope_cache_write(qkv: torch.Tensor, q_out: torch.Tensor, cos_sin: Optional[torch.Tensor],
                     positions: torch.Tensor, dest: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                     v_cache: Optional[torch.Tensor], nh: int, nkv: int, hd: int, page_size: int,
                     write_kv: bool = True) -> None:
    T = q_out.shape[0]
    width = (nh + 2 * nkv) * hd if write_kv else nh * hd
    _need(qkv, "qkv")
    if qkv.shape[0] != T or qkv.shape[1] < width:
        raise KernelError(f"rope: qkv shape {tuple(qkv.shape)} does not hold {T} rows of width {width}")
    _need(q_out, "q_out", None, (T, nh * hd))
    _need(positions, "positions", torch.int32, (T,))
    rotate = cos_sin is not None
    if rotate:
        _need(cos_sin, "rope table", torch.float32)
        if cos_sin.shape[1:] != (hd // 2, 2):
            raise KernelError(f"rope: table shape {tuple(cos_sin.shape)} does not fit head_dim {hd}")
    if write_kv:
        _need(dest, "cache rows", torch.int32, (T,))
        _need(k_cache, "k cache", q_out.dtype)
        _need(v_cache, "v cache", q_out.dtype)
    _check(_lib("rope_cache").jb_rope_cache_write(
        _ptr(qkv), qkv.shape[1], dtype_code(qkv.dtype), _ptr(q_out), dtype_code(q_out.dtype), _ptr(cos_sin),
        _ptr(positions), _ptr(dest), _ptr(k_cache), _ptr(v_cache),
        T, nh, nkv, hd, page_size, int(rotate), int(write_kv), _stream()), "rope_cache_write")


# -- float32 matrix product and attention ------------------------------------------
def gemm_f32(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, accumulate: bool = False, label: str = "") -> None:
    """y[T, N] (+)= x[T, K] . w[N, K]^T in true float32 (`label`: what a profile of a step calls this product)"""
    T, K = x.shape
    N = w.shape[0]
    _need(x, "gemm x", torch.float32)
    _need(w, "gemm w", torch.float32, (N, K))
    _need(y, "gemm y", torch.float32, (T, N))
    _check(_lib("gemm_f32").jb_gemm_f32(_ptr(x), _ptr(w), _ptr(y), T, N, K, K, N, int(accumulate), _stream()),
           "gemm_f32 " + label if label else "gemm_f32")


def attention_f32(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                  block_table: torch.Tensor, token_slot: torch.Tensor, positions: torch.Tensor,
                  nh: int, nkv: int, hd: int, page_size: int, window: int, scale: float) -> None:
    T = q.shape[0]
    _need(q, "attention q", torch.float32, (T, nh * hd))
    _need(out, "attention out", torch.float32, (T, nh * hd))
    _need(k_cache, "k cache", torch.float32)
    _need(v_cache, "v cache", torch.float32)
    _need(block_table, "block table", torch.int32)
    _need(token_slot, "token slots", torch.int32, (T,))
    _need(positions, "positions", torch.int32, (T,))
    _check(_lib("attention_f32").jb_attention_f32(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), _ptr(token_slot), _ptr(positions),
        T, nh, nkv, hd, page_size, block_table.shape[1], int(window), scale, _stream()),
        "attention_f32")


# -- bfloat16 tensor-core matrix product --------------------------------------------
_status = {}
SM_COUNT_TARGET = 296      # CTAs wanted in flight for a weight-streaming product (two per SM)


_bound_device = []


def bind_device(device: torch.device) -> None:
    """One process drives one GPU: the kernel libraries set their kernels up (shared-memory limits, occupancy,
    SM count) for the device of their first launch and keep that.  The first model names the device; a model
    on another device is refused here, not at some launch."""
    index = torch.device(device).index
    index = torch.cuda.current_device() if index is None else index
    if not _bound_device:
        _bound_device.append(index)
    elif _bound_device[0] != index:
        raise KernelError(f"this process already runs its kernels on cuda:{_bound_device[0]}; a model on "
                          f"cuda:{index} needs a process of its own (the library drives one GPU per process)")


def kernel_status(device: torch.device) -> torch.Tensor:
    """Device int that a kernel sets when one of its bounded waits ran out."""
    st = _status.get(device)
    if st is None:
        st = torch.zeros(1, dtype=torch.int32, device=device)
        _status[device] = _status[st.device] = st       # "cuda" and "cuda:0" name the same word
    return st


def check_kernel_status(device: torch.device) -> None:
    """Synchronises; raises if a tensor-core kernel gave up on a wait."""
    code = int(kernel_status(device).item())
    if code != 0:
        kernel_status(device).zero_()
        who = {1: "TMA producer", 2: "MMA issuer", 3: "epilogue"}.get(code % 10, "?")
        raise KernelError(f"a tensor-core kernel timed out waiting on an mbarrier ({who}, code {code})")


class PackedWeight:
    """A [rows, cols] bfloat16 matrix laid out for the tensor-core products: tiles of 128 rows x 64 columns,
    each one contiguous, zero-padded and already swizzled 16 KB block, stored [row tile][k tile]
    (`pack_weight`).  A stage of a product then reads its weights as one sequential block of HBM.
    `up_tile_offset` > 0 marks a gated pair: the gate matrix's row tiles first, the up matrix's row tiles
    from there on (`rows` counts one of the two)."""

    def __init__(self, tiles: torch.Tensor, rows: int, cols: int, up_tile_offset: int = 0):
        self.tiles, self.rows, self.cols, self.up_tile_offset = tiles, int(rows), int(cols), int(up_tile_offset)

    @property
    def n_tiles(self) -> int:
        return self.tiles.shape[0] * self.tiles.shape[1]

    @property
    def device(self):
        return self.tiles.device

    def nbytes(self) -> int:
        return self.tiles.numel() * 2

    def first_rows(self, rows: int) -> "PackedWeight":
        """The matrix of the first `rows` rows (shares storage; a last tile may hold further rows, which
        the product's epilogue leaves out)."""
        if rows > self.rows or self.up_tile_offset:
            raise KernelError(f"first_rows({rows}) of a packed matrix of {self.rows} rows")
        return PackedWeight(self.tiles[: (rows + 127) // 128], rows, self.cols)

    def stacked(self) -> "PackedWeight":
        """A gated pair as the plain matrix of its row tiles: the gate rows (padded to whole tiles of 128),
        then the up rows from row 128 * up_tile_offset on (shares storage)."""
        if not self.up_tile_offset:
            raise KernelError("stacked(): the weight is no gated pair")
        return PackedWeight(self.tiles, self.tiles.shape[0] * 128, self.cols)


def pack_weight(w: torch.Tensor) -> PackedWeight:
    """Row-major bfloat16 [N, K] (K a multiple of 8) -> PackedWeight."""
    _need(w, "weight to pack", torch.bfloat16)
    if w.dim() != 2 or w.shape[1] % 8:
        raise KernelError(f"pack_weight: a matrix whose width is a multiple of 8 is needed, got {tuple(w.shape)}")
    N, K = w.shape
    tiles = torch.empty(((N + 127) // 128, (K + 63) // 64, 128, 64), dtype=torch.bfloat16, device=w.device)
    _check(_lib("elementwise").jb_pack_weight_bf16(_ptr(w), N, K, _ptr(tiles), _stream()), "pack_weight")
    return PackedWeight(tiles, N, K)


def pack_gated(gate: torch.Tensor, up: torch.Tensor) -> PackedWeight:
    """Gate and up matrices of equal shape as one PackedWeight (gate tiles, then up tiles)."""
    if gate.shape != up.shape:
        raise KernelError(f"pack_gated: shapes {tuple(gate.shape)} and {tuple(up.shape)} differ")
    g, u = pack_weight(gate), pack_weight(up)
    return PackedWeight(torch.cat([g.tiles, u.tiles], dim=0), gate.shape[0], gate.shape[1], g.tiles.shape[0])


# JANUS_DETERMINISTIC=1 (or `set_deterministic(True)` before a model is built): the slices of a cut K are
# summed in the fixed order of the slices instead of by atomic adds in the order they happen to finish, so the
# same requests give the same bits.  Every slice leaves its tile in scratch; the one that arrives last at the
# output tile's ticket adds them up (single-CTA kernel; CTA pairs then run uncut).
_deterministic = [os.environ.get("JANUS_DETERMINISTIC", "0") == "1"]


def set_deterministic(flag: bool) -> None:
    """Switch cutting of K (atomic adds) off or on for products launched from now on; decode steps that an
    engine has already captured into CUDA graphs keep what they were captured with."""
    _deterministic[0] = bool(flag)
    gemm_plan.cache_clear()


def is_deterministic() -> bool:
    return _deterministic[0]


ORDERED_SCRATCH_MAX_BYTES = 256 << 20
_ORDERED_TICKETS = 1 << 16
_ordered_scratch = {}     # device -> (partials, tickets); outgrown buffers stay alive for captured graphs
_ordered_retired = []


def _ordered_buffers(device: torch.device, floats: int):
    """Scratch for ordered sums of `floats` floats on `device` (None if that is more than the cap)."""
    if floats * 4 > ORDERED_SCRATCH_MAX_BYTES:
        return None
    have = _ordered_scratch.get(device)
    if have is None or have[0].numel() < floats:
        size = max(floats, 2 * have[0].numel() if have is not None else (8 << 20) // 4)
        size = min(size, ORDERED_SCRATCH_MAX_BYTES // 4)
        tickets = have[1] if have is not None else torch.zeros(_ORDERED_TICKETS, dtype=torch.int32, device=device)
        if have is not None:
            _ordered_retired.append(have[0])
        have = (torch.empty(size, dtype=torch.float32, device=device), tickets)
        _ordered_scratch[device] = have
    return have


def gated_runs_unfused(T: int, I: int) -> bool:
    """Whether a SiLU-gated product of I features runs as a plain product of the stacked gate and up rows
    into float32 and an activation kernel: decode-sized steps of narrow layers, where the fused kernel's
    tiles (128 features, gate and up rows together) fill less than half of the SMs.  Measured at 8192
    features (64 tiles): 13.6 us against 15.1 at 8 tokens, 17.6 against 21.5 at 64; at 13824 and 14336
    features the fused kernel is faster (45.5 against 45.8 to 51.9, 37.1 against 40.0 to 44.6)."""
    return _GATED_UNFUSED and T <= 64 and 2 * ((I + 127) // 128) <= SM_COUNT_TARGET // 2


_GATED_UNFUSED = os.environ.get("JANUS_GATED_UNFUSED", "1") != "0"


def split_k_for(T: int, N: int, K: int) -> int:
    """How many slices of K an adding product (mode "add", or a float32 "store" run as clear + add) is cut
    into; 1 when it is not cut."""
    return gemm_plan(T, N, K, "add")[1]


# token counts from which the CTA-pair kernel (cta_group::2, 256-row weight tiles) may run a product;
# JANUS_GEMM_PAIR=0 keeps every product on the single-CTA kernel
GEMM_PAIR_MIN_TOKENS = int(os.environ.get("JANUS_GEMM_PAIR_MIN_TOKENS", "65"))
_GEMM_PAIR = os.environ.get("JANUS_GEMM_PAIR", "1") != "0"
# token counts from which the q/k/v projection with rotation and cache append in its epilogue runs
QKV_FUSED_MIN_TOKENS = int(os.environ.get("JANUS_QKV_FUSED_MIN_TOKENS", "512"))

# Constants of the cost estimate in `gemm_plan`.  They were fitted so that the estimate picks the fastest
# of the alternatives (the single-CTA kernel with K in 1, 2, 3, 4, 6 or 8 slices; CTA pairs with K in 1, 2,
# 3, 4 or 6) as measured on a B200 for the four products of 1B-, 8B-, 13B- and 70B-sized layers at 72 to
# 4096 tokens: the pick is 0.4 % slower than the best alternative on average.  They rank alternatives; they
# are no forecast of a time.
_PLAN_SM_FLOPS_PER_US = 6.09e6      # tensor-core rate of one SM on single-CTA tiles, flop per microsecond
_PLAN_SM_FILL_BYTES_PER_US = 1.99e5  # operand bytes one SM takes in per microsecond
_PLAN_TILE_US = 0.0                 # per tile of the single-CTA kernel
_PLAN_PAIR_STEP_US = 0.461          # one 256 x 256 x 64 step of a CTA pair
_PLAN_PAIR_TILE_US = 4.18           # per tile of a CTA pair: first loads, epilogue
_PLAN_HBM_BYTES_PER_US = 6.68e6     # the weight stream
_PLAN_US_PER_ADD = 5.14e-7          # one float32 add of a slice of K into the output, single-CTA kernel
_PLAN_PAIR_US_PER_ADD = 4.26e-7     # the same, CTA pairs
_PLAN_SPLITS = (1, 2, 3, 4, 6, 8)
_PLAN_DECODE_MAX_SPLIT = 24
_PLAN_DECODE_STEPS_PER_ADD = 1e-4   # adds of a 128-row tile's token, in steps along K (fitted: 60 measured cases)
_PLAN_PAIR_SPLITS = (1, 2, 3, 4, 6)
_PLAN_ORDERED_TILE_US = 3.0         # deterministic mode: fence, ticket and ordered sum of a tile of a cut K
_PLAN_TAIL_MIN_K = 32               # k-tiles a slice of a last wave's tile has at least (measured: the o projection
                                    # of 8B layers, 64 k-tiles, loses 4 % with slices of 16; the down projection, 224, gains 12 %)


def gemm_plan(T: int, N: int, K: int, mode: str, allow_pairs: bool = True) -> Tuple[bool, int]:
    """(CTA pairs?, slices of K): see `gemm_plan_whole`, which also says how many tiles stay uncut."""
    return gemm_plan_whole(T, N, K, mode, allow_pairs)[:2]


def _plan_cache_clear() -> None:
    gemm_plan_whole.cache_clear()


gemm_plan.cache_clear = _plan_cache_clear


@functools.lru_cache(maxsize=4096)
def gemm_plan_whole(T: int, N: int, K: int, mode: str, allow_pairs: bool = True) -> Tuple[bool, int, int]:
    """Which kernel runs x[T, K] . w[N, K]^T and into how many slices of K it is cut: (CTA pairs?, slices).

    Up to 64 tokens the product streams its weights: the single-CTA kernel, with K cut so that the waves of
    tiles over the SMs x the steps of a slice are fewest (only a product that adds can be cut; its slices
    meet by atomic adds): 4096 x 4096 makes 32 tiles, and 13 slices of 5 steps in 3 waves beat 9 of 8 in 2.
    Above, the choice is by an estimate of the time: waves of tiles over the SMs x (steps along K x the
    time of a step, tensor-core bound or bound by what an SM takes in per step, + a tile's fixed cost), not
    below the time of the weight stream, plus the atomic adds of a cut K.  Few output tiles (a 4096 x 4096
    matrix and 256 tokens make 32) leave most SMs idle unless K is cut; CTA pairs halve the operand bytes
    per flop and win once their 256 x 256 tiles fill the SMs."""
    tiles_w = (N + 127) // 128
    k_tiles = (K + 63) // 64
    sms = SM_COUNT_TARGET // 2
    ordered = _deterministic[0]     # slices are summed in a fixed order: the single-CTA kernel can, CTA pairs cannot
    if T <= 64:
        if mode != "add" or tiles_w >= sms:
            return False, 1, 0   # a wave of tiles or more streams weights on every SM as it is
        # the critical path in steps along K: waves of tiles over the SMs x steps of a slice; a little per add
        best = (float("inf"), 1)
        for split in range(1, max(1, min(k_tiles // 4, _PLAN_DECODE_MAX_SPLIT)) + 1):
            waves = (tiles_w * split + sms - 1) // sms
            if ordered and split > 1 and waves > 1:
                break     # an ordered sum costs a tile a fence and a ticket (about 3 us): one tile per SM at most
            cost = waves * ((k_tiles + split - 1) // split) + _PLAN_DECODE_STEPS_PER_ADD * split * T * tiles_w
            if cost < best[0] - 1e-9:
                best = (cost, split)
        return False, best[1], 0
    gated = mode == "swiglu"
    w_rows = 2 * N if gated else N
    stream = w_rows * K * 2 / _PLAN_HBM_BYTES_PER_US
    # token tile of the single-CTA kernel (a gated product's two accumulators leave room for 256 tokens in one
    # buffer only, which serves where a CTA has one tile: up to 256 tokens)
    bn = 128 if (T <= 128 or (gated and T > 256)) else 256
    stage_rows = 256 if gated else 128                      # weight rows a step brings in
    step = max(2.0 * stage_rows * bn * 64 / _PLAN_SM_FLOPS_PER_US,
               (stage_rows + bn) * 64 * 2 / _PLAN_SM_FILL_BYTES_PER_US)
    best = (float("inf"), False, 1, 0)
    for split in (_PLAN_SPLITS if mode == "add" else (1,)):
        if split > 1 and split > k_tiles // 4:
            break
        tiles = tiles_w * ((T + bn - 1) // bn) * split
        waves = (tiles + sms - 1) // sms
        cost = max(waves * (((k_tiles + split - 1) // split) * step + _PLAN_TILE_US), stream)
        if split > 1:
            cost += _PLAN_US_PER_ADD * T * N * split + (_PLAN_ORDERED_TILE_US * waves if ordered else 0.0)
        best = min(best, (cost, False, split, 0))
    if allow_pairs and _GEMM_PAIR and T >= GEMM_PAIR_MIN_TOKENS:
        clusters = ((T + 255) // 256) * (tiles_w if gated else (N + 255) // 256)
        for split in (_PLAN_PAIR_SPLITS if mode == "add" and not ordered else (1,)):
            if split > 1 and split > k_tiles // 4:
                break
            waves = (clusters * split + sms // 2 - 1) // (sms // 2)
            cost = max(waves * (((k_tiles + split - 1) // split) * _PLAN_PAIR_STEP_US + _PLAN_PAIR_TILE_US), stream)
            if split > 1:
                cost += _PLAN_PAIR_US_PER_ADD * T * N * split
            best = min(best, (cost, True, split, 0))
        pairs = sms // 2
        whole, tail = clusters // pairs * pairs, clusters % pairs
        if mode == "add" and not ordered and whole and tail:
            # more than a wave of tiles and a last wave that is not full: only that wave's tiles are cut, into
            # slices of at least _PLAN_TAIL_MIN_K k-tiles (shorter pieces are all epilogue)
            for split in _PLAN_PAIR_SPLITS[1:] + (8,):
                per = (k_tiles + split - 1) // split
                if per < _PLAN_TAIL_MIN_K:
                    break
                rounds = (tail * split + pairs - 1) // pairs
                cost = max(whole // pairs * (k_tiles * _PLAN_PAIR_STEP_US + _PLAN_PAIR_TILE_US)
                           + rounds * (per * _PLAN_PAIR_STEP_US + _PLAN_PAIR_TILE_US), stream)
                cost += _PLAN_PAIR_US_PER_ADD * T * N * split * tail / clusters
                best = min(best, (cost, True, split, whole))
    return best[1], best[2], best[3]


def _defines_from_env(name: str) -> dict:
    """Build-time overrides of a kernel's tuning macros for experiments, read once when this module loads,
    e.g. JANUS_GEMM_DEFINES="JB_RING_KB=104,JB_MAX_STAGES=6"; none by default."""
    text = os.environ.get(name, "")
    return {k.strip(): int(v) for k, v in (item.split("=") for item in text.split(",") if item.strip())}


def _defines_key(defines: Optional[dict]):
    return tuple(sorted(defines.items())) if defines else None


_GEMM_DEFINES = _defines_from_env("JANUS_GEMM_DEFINES") or None
_PAIR_DEFINES = _defines_from_env("JANUS_GEMM_PAIR_DEFINES") or None
_ATTN_TC_DEFINES = _defines_from_env("JANUS_ATTN_TC_DEFINES")
_ATTN_DEFINES = _defines_from_env("JANUS_ATTN_DEFINES")
_ATTN_TC = os.environ.get("JANUS_ATTN_TC", "1") != "0"     # 0: prompts attend on the mma.sync kernel


def gemm_bf16(x: torch.Tensor, w: PackedWeight, y: torch.Tensor, mode: str = "store",
              split_k: Optional[int] = None, pair: Optional[bool] = None, whole_tiles: int = 0,
              label: str = "") -> None:
    """bf16 x[T, K] . w[N, K]^T on tcgen05 with float32 accumulation; w packed (`pack_weight`).
    mode "store": y[T, N] = result (bf16 or float32 by y's dtype);
    mode "add":   y[T, N] += result, y float32 (K may be split, sums meet by atomic adds);
    mode "swiglu": w a gated pair (`pack_gated`), y[T, N] = silu(gate) * up in bf16.
    `split_k`, `pair`, `whole_tiles`: as `gemm_plan_whole` picks them unless given (`whole_tiles`: CTA pairs
    only, the first so many 256 x 256 output tiles of an adding product stay uncut)."""
    T, K = x.shape
    _need(x, "gemm x", torch.bfloat16)
    _need(y, "gemm y")
    if not isinstance(w, PackedWeight):
        raise KernelError("gemm: the weight must be packed (ops.pack_weight / ops.pack_gated)")
    if w.cols != K:
        raise KernelError(f"gemm: weight of {w.rows} x {w.cols} does not fit K = {K}")
    N = w.rows
    if mode == "swiglu":
        code, want = 3, torch.bfloat16
        if not w.up_tile_offset:
            raise KernelError("gemm swiglu: the weight is no gated pair (ops.pack_gated)")
    else:
        if w.up_tile_offset:
            raise KernelError(f"gemm {mode}: the weight is a gated pair")
        if mode == "add":
            code, want = 2, torch.float32
        elif mode == "store":
            code, want = (1, torch.float32) if y.dtype == torch.float32 else (0, torch.bfloat16)
        else:
            raise KernelError(f"gemm: unknown mode {mode!r}")
    if y.dtype != want or tuple(y.shape) != (T, N):
        raise KernelError(f"gemm {mode}: output must be {want} [{T}, {N}], got {y.dtype} {tuple(y.shape)}")
    if split_k is None:
        if pair is not True:
            pair, split_k, whole_tiles = gemm_plan_whole(T, N, K, mode, allow_pairs=pair is not False)
        else:
            split_k = 1
        if code != 2:
            split_k = 1          # a storing product cut along K is the caller's clear + "add"
    elif pair is None:
        pair = False
    if pair:
        _check(_lib("gemm_bf16_tc2", _defines_key(_PAIR_DEFINES), _PAIR_DEFINES).jb_gemm_bf16_pair(
            _ptr(x), _ptr(w.tiles), w.n_tiles, w.up_tile_offset, _ptr(y), T, N, K, N, code,
            int(split_k), int(whole_tiles), _ptr(kernel_status(x.device)), _stream()),
            "gemm_bf16_pair " + label if label else "gemm_bf16_pair")
        return
    partials = tickets = None
    if split_k > 1 and _deterministic[0]:
        bn = 16 if T <= 16 else 32 if T <= 32 else 64 if T <= 64 else 128 if T <= 128 else 256
        k_tiles = (K + 63) // 64
        per = (k_tiles + split_k - 1) // split_k
        slices = (k_tiles + per - 1) // per
        out_tiles = ((N + 127) // 128) * ((T + bn - 1) // bn)
        scratch = _ordered_buffers(x.device, out_tiles * slices * bn * 128) if out_tiles <= _ORDERED_TICKETS else None
        if scratch is None:
            split_k = 1          # too much scratch: K whole
        else:
            partials, tickets = scratch
    _check(_lib("gemm_bf16_tc", _defines_key(_GEMM_DEFINES), _GEMM_DEFINES).jb_gemm_bf16(
        _ptr(x), _ptr(w.tiles), w.n_tiles, w.up_tile_offset, _ptr(y), T, N, K, N, code,
        int(split_k), _ptr(partials), 0 if partials is None else partials.numel(), _ptr(tickets),
        0 if tickets is None else tickets.numel(), _ptr(kernel_status(x.device)), _stream()),
        "gemm_bf16 " + label if label else "gemm_bf16")


def gemm_qkv_rope_supported(T: int, hd: int) -> bool:
    """Whether the fused projection below takes this step: prompt-sized token counts and a head size that
    divides the kernel's 256 columns with half-heads of whole 16-column loads."""
    return _GEMM_PAIR and _QKV_FUSED and T >= QKV_FUSED_MIN_TOKENS and hd in (32, 64, 128, 256)


_QKV_FUSED = os.environ.get("JANUS_QKV_FUSED", "1") != "0"   # 0: projection, then rotation and cache append apart


def gemm_qkv_rope_cache(x: torch.Tensor, w: PackedWeight, q_out: torch.Tensor, cos_sin: torch.Tensor,
                        positions: torch.Tensor, dest: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                        nh: int, nkv: int, hd: int, page_size: int) -> None:
    """The stacked q/k/v projection x[T, K] . w[(nh + 2 nkv) hd, K]^T on CTA pairs with its consumers fused
    into the epilogue: q and k rotated by cos_sin[positions], q to q_out[T, nh hd], k and v to the paged
    cache at rows dest, all bfloat16 from the float32 accumulators."""
    T, K = x.shape
    _need(x, "qkv x", torch.bfloat16)
    if not isinstance(w, PackedWeight) or (w.rows, w.cols) != ((nh + 2 * nkv) * hd, K) or w.up_tile_offset:
        raise KernelError(f"qkv: a packed weight of {(nh + 2 * nkv) * hd} x {K} is needed")
    _need(q_out, "q_out", torch.bfloat16, (T, nh * hd))
    _need(cos_sin, "rope table", torch.float32)
    if cos_sin.shape[1:] != (hd // 2, 2):
        raise KernelError(f"qkv: table shape {tuple(cos_sin.shape)} does not fit head_dim {hd}")
    _need(positions, "positions", torch.int32, (T,))
    _need(dest, "cache rows", torch.int32, (T,))
    _need(k_cache, "k cache", torch.bfloat16)
    _need(v_cache, "v cache", torch.bfloat16)
    if k_cache.shape[1:] != (nkv, page_size, hd) or v_cache.shape != k_cache.shape:
        raise KernelError(f"qkv: cache shape {tuple(k_cache.shape)} is not [pages, {nkv}, {page_size}, {hd}]")
    _check(_lib("gemm_bf16_tc2", _defines_key(_PAIR_DEFINES), _PAIR_DEFINES).jb_gemm_bf16_pair_qkv_rope(
        _ptr(x), _ptr(w.tiles), w.n_tiles, T, K, _ptr(q_out), _ptr(k_cache), _ptr(v_cache),
        _ptr(cos_sin), _ptr(positions), _ptr(dest),
        nh, nkv, hd, page_size, _ptr(kernel_status(x.device)), _stream()), "gemm_bf16_pair_qkv_rope")


# -- sampling -----------------------------------------------------------------------
def sample(logits: torch.Tensor, out_ids: torch.Tensor, temperature: float, top_k: int, top_p: float,
           repetition_penalty: float, counts: Optional[torch.Tensor], count_rows: Optional[torch.Tensor],
           seed: int, seq_ids: torch.Tensor, steps: torch.Tensor, feedback: Optional[torch.Tensor] = None) -> None:
    B, V = logits.shape
    _need(logits, "logits", torch.float32)
    _need(out_ids, "sampled ids", torch.int32, (B,))
    _need(seq_ids, "sequence ids", torch.int32, (B,))
    _need(steps, "step counters", torch.int32, (B,))
    if count_rows is not None:
        _need(count_rows, "rows' slots", torch.int32, (B,))
    if feedback is not None:
        _need(feedback, "token feedback", torch.int32)
    if counts is not None:
        _need(counts, "token counts", torch.int32)
        if counts.shape[1] != V:
            raise KernelError("sample: counts width differs from the vocabulary")
    _check(_lib("sampling").jb_sample(
        _ptr(logits), B, V, _ptr(out_ids), temperature, int(top_k), top_p,
        repetition_penalty, _ptr(counts), _ptr(count_rows),
        seed & ((1 << 64) - 1), _ptr(seq_ids), _ptr(steps), _ptr(feedback), _stream()),
        "sample")


# -- bfloat16 attention (one library per head size) -----------------------------------
ATTENTION_MAX_HEAD_DIM = 256      # every attention kernel, float32 and bfloat16
ATTENTION_BF16_MAX_GROUP = 64     # query heads per kv head of the mma.sync prompt kernel (a row tile holds 64 rows)


def _attention_lib(hd: int):
    if hd % 8 or not 8 <= hd <= 256:
        raise KernelError(f"attention_bf16: head_dim {hd} is not a multiple of 8 in [8, 256]")
    return _lib("attention_bf16", int(hd), lambda h: dict({"JB_HEAD_DIM": h}, **_ATTN_DEFINES))


def attention_bf16_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                           block_table: torch.Tensor, q_start: torch.Tensor, kv_len: torch.Tensor,
                           n_seqs: int, max_q_len: int, nh: int, nkv: int, hd: int, page_size: int,
                           window: int, scale: float) -> None:
    """Causal attention of each sequence's new tokens (the last q_len positions of
    its kv_len) over its cached keys."""
    T = q.shape[0]
    _need(q, "attention q", torch.bfloat16, (T, nh * hd))
    _need(out, "attention out", torch.bfloat16, (T, nh * hd))
    _need(k_cache, "k cache", torch.bfloat16)
    _need(v_cache, "v cache", torch.bfloat16)
    _need(block_table, "block table", torch.int32)
    _need(q_start, "q_start", torch.int32, (n_seqs + 1,))
    _need(kv_len, "kv_len", torch.int32, (n_seqs,))
    _check(_attention_lib(hd).jb_attention_bf16_prefill(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), _ptr(q_start), _ptr(kv_len),
        n_seqs, max_q_len, nh, nkv, hd, page_size, block_table.shape[1], int(window), scale,
        _stream()), "attention_bf16_prefill")


# Constants of the estimate in `decode_splits_for` (microseconds, bytes per microsecond), read off measurements
# of the decode kernel at head sizes 64 and 128 (1 to 64 sequences of 1,024 to 4,000 keys, 8 and 40 kv heads,
# 1 to 8 splits): they rank split counts, they forecast no time.
_SPLIT_CTA_US = 3.0                 # a CTA's start, its queries, its last exchange and write
_SPLIT_PAGE_US = {64: 0.6, 128: 0.85}   # a CTA alone walks a page of 64 keys in this time (head size up to 64 / above)
_SPLIT_HBM_BYTES_PER_US = 6.2e6
_SPLIT_COMBINE_US = 3.0             # the kernel that joins the splits, plus 0.05 a split
_SPLIT_SHARED_SM = 0.2              # a CTA that shares its SM with another walks its pages this much slower
_SPLIT_CHOICES = (1, 2, 3, 4, 6, 8, 12, 16, 24, 32)


def _decode_ctas_per_sm(head_dim: int, ctas: int, pages_per_cta: int) -> int:
    """CTAs of the decode kernel that share an SM: its ring of pages is picked at the launch (in step with
    `decode_stages_for` of csrc/attention_bf16.cu): three pages for large heads (two CTAs an SM at head size
    128); small heads take two pages when there are more CTAs than fit at once (five an SM at head size 64),
    five pages for few CTAs of many pages (two an SM), else three (three an SM)."""
    ld = (head_dim + 15) // 16 * 16 + 8

    def fit(stages: int) -> int:
        smem = 18 * ld * 2 + max(2 * stages * 64 * ld * 2, (4 * 16 * (head_dim + 8) + 128) * 4)
        return max(1, min(16, 228 * 1024 // (smem + 1024)))

    if head_dim > 64:
        return fit(3)
    sms = SM_COUNT_TARGET // 2
    if ctas > sms * fit(3):
        return fit(2)
    if ctas <= sms * fit(5) and pages_per_cta >= 8:
        return fit(5)
    return fit(3)


@functools.lru_cache(maxsize=4096)
def decode_splits_for(n_seqs: int, nkv_blocks: int, max_kv_len: int, page_size: int, head_dim: int = 128) -> int:
    """Splits of the key range per (sequence, kv head), from an estimate of the kernel's time for each count.

    A launch is `n_seqs * nkv_blocks * splits` CTAs of about `pages / splits` pages each; as many CTAs as fit the
    SMs run at once (a wave).  A wave takes as long as its bytes need at the memory's rate, but no less than one
    CTA needs to walk its pages (a little longer where CTAs share an SM); the waves add up, and more than one
    split costs the kernel that joins them.  So few sequences want many splits (one sequence of 2,080 keys: 16), a batch that fills the SMs wants
    none (64 sequences over 8 kv heads: 1), and a batch that overfills them a little wants its CTAs small, so
    that the last wave is short (8 sequences over 40 kv heads, 320 CTAs for 296 places: 4 splits, 62 us against
    76 us uncut).  `max_kv_len` is the bound a step was laid out for (a power of two of pages); sequences are
    taken to be three quarters of it."""
    cap_pages = max(1, (max_kv_len + page_size - 1) // page_size)
    pages = max(1, (3 * cap_pages + 3) // 4)
    base = max(1, n_seqs * nkv_blocks)
    sms = SM_COUNT_TARGET // 2
    page_us = _SPLIT_PAGE_US[64 if head_dim <= 64 else 128]
    page_bytes = page_size * head_dim * 2 * 2
    best = (float("inf"), 1)
    for splits in _SPLIT_CHOICES:
        if splits > 1 and splits > max(1, cap_pages // 2):
            break
        per = (pages + splits - 1) // splits
        ctas = base * splits
        places = sms * _decode_ctas_per_sm(head_dim, ctas, per)
        alone = _SPLIT_CTA_US + per * page_us

        def wave(n: int) -> float:      # n CTAs at once: on how many SMs, at the memory's rate or a CTA's own pace
            sharing = 1.0 + _SPLIT_SHARED_SM * ((n + sms - 1) // sms - 1)
            return max(alone * sharing, n * per * page_bytes / _SPLIT_HBM_BYTES_PER_US)

        full, rest = divmod(ctas, places)
        cost = full * wave(places) + (wave(rest) if rest else 0.0)
        if splits > 1:
            cost += _SPLIT_COMBINE_US + 0.05 * splits
        if cost < best[0] - 1e-9:
            best = (cost, splits)
    return best[1]


def attention_bf16_decode(q: Optional[torch.Tensor], k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                          block_table: torch.Tensor, kv_len: torch.Tensor, nh: int, nkv: int, hd: int,
                          page_size: int, window: int, scale: float, workspace, max_kv_len: int,
                          n_splits: Optional[int] = None, qkv: Optional[torch.Tensor] = None,
                          cos_sin: Optional[torch.Tensor] = None, dest: Optional[torch.Tensor] = None,
                          write_kv: bool = True) -> None:
    """One new token per sequence (its last position) over its cached keys.

    Either `q` (rotated bf16 queries; the cache already holds the new token), or `qkv`: the
    projection's float32 output [B, (nh + 2 nkv) hd] (or [B, nh hd] with write_kv False), which the
    kernel rotates with `cos_sin` (None: no rotation), appends to the cache at rows `dest` and uses."""
    B = out.shape[0]
    _need(out, "attention out", torch.bfloat16, (B, nh * hd))
    _need(k_cache, "k cache", torch.bfloat16)
    _need(v_cache, "v cache", torch.bfloat16)
    _need(block_table, "block table", torch.int32)
    _need(kv_len, "kv_len", torch.int32, (B,))
    n_rb = (nh // nkv + 15) // 16
    if n_splits is None:
        n_splits = decode_splits_for(B, nkv * n_rb, max_kv_len, page_size, hd)
    part_o = part_ml = None
    if n_splits > 1:
        part_o = workspace.get("attn_part_o", (B * nh * n_splits * hd,), torch.float32)
        part_ml = workspace.get("attn_part_ml", (B * nh * n_splits * 2,), torch.float32)
    lib = _attention_lib(hd)
    kernels = 2 if n_splits > 1 else 1
    if qkv is None:
        _need(q, "attention q", torch.bfloat16, (B, nh * hd))
        _check(lib.jb_attention_bf16_decode(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(block_table),
            _ptr(kv_len), B, nh, nkv, hd, page_size, block_table.shape[1], int(window), scale,
            int(n_splits), _stream()), "attention_bf16_decode", kernels=kernels)
        return
    _need(qkv, "qkv", torch.float32)
    width = (nh + 2 * nkv) * hd if write_kv else nh * hd
    if qkv.shape[0] != B or qkv.shape[1] < width:
        raise KernelError(f"attention decode: qkv shape {tuple(qkv.shape)} does not hold {B} rows of width {width}")
    if cos_sin is not None:
        _need(cos_sin, "rope table", torch.float32)
        if cos_sin.shape[1:] != (hd // 2, 2):
            raise KernelError(f"attention decode: table shape {tuple(cos_sin.shape)} does not fit head_dim {hd}")
    if write_kv:
        _need(dest, "cache rows", torch.int32, (B,))
    _check(lib.jb_attention_bf16_decode_fused(
        _ptr(qkv), qkv.shape[1], _ptr(cos_sin), _ptr(dest), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(part_o),
        _ptr(part_ml), _ptr(block_table), _ptr(kv_len), B, nh, nkv, hd, page_size, block_table.shape[1], int(window),
        scale, int(n_splits), int(write_kv), _stream()), "attention_bf16_decode_fused", kernels=kernels)


# -- tcgen05 prefill attention (head sizes up to 256 in steps of 8, up to 128 query heads per kv head) -----
ATTENTION_TC_MAX_HEAD_DIM = 256


def attention_tc_supported(nh: int, nkv: int, hd: int) -> bool:
    g = nh // max(nkv, 1)
    return (_ATTN_TC and 0 < hd <= ATTENTION_TC_MAX_HEAD_DIM and hd % 8 == 0 and nkv > 0 and nh % nkv == 0
            and g <= 128)


def _attention_tc_row(hd: int) -> int:
    """The build that takes head size `hd`: rows of 64, 128 or 256 dims in shared memory."""
    return 64 if hd <= 64 else 128 if hd <= 128 else 256


def attention_tc_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                         block_table: torch.Tensor, q_start: torch.Tensor, kv_len: torch.Tensor,
                         n_seqs: int, max_q_len: int, nh: int, nkv: int, hd: int, page_size: int,
                         window: int, scale: float) -> None:
    """As attention_bf16_prefill, on the tcgen05 tensor cores."""
    T = q.shape[0]
    _need(q, "attention q", torch.bfloat16, (T, nh * hd))
    _need(out, "attention out", torch.bfloat16, (T, nh * hd))
    _need(k_cache, "k cache", torch.bfloat16)
    _need(v_cache, "v cache", torch.bfloat16)
    _need(block_table, "block table", torch.int32)
    _need(q_start, "q_start", torch.int32, (n_seqs + 1,))
    _need(kv_len, "kv_len", torch.int32, (n_seqs,))
    if tuple(k_cache.shape[1:]) != (nkv, page_size, hd) or k_cache.shape != v_cache.shape:
        raise KernelError(f"attention_tc: cache shape {tuple(k_cache.shape)} does not fit [pages, {nkv}, {page_size}, {hd}]")
    _check(_lib("attention_tc", _attention_tc_row(hd),
                lambda h: dict({"JB_HEAD_DIM": h}, **_ATTN_TC_DEFINES)).jb_attention_tc_prefill(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), _ptr(q_start), _ptr(kv_len),
        T, k_cache.shape[0], n_seqs, max_q_len, nh, nkv, hd, page_size, block_table.shape[1], int(window),
        scale, _ptr(kernel_status(q.device)), _stream()), "attention_tc_prefill")
