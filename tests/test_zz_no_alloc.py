"""The decode-attention entry point that allocates nothing
(`jb_attention_bf16_decode_noalloc`, declared in csrc/attention_bf16_noalloc.h).

Some users of this library may not call cudaMalloc where they call us: their
device memory was planned or handed out beforehand, or an allocator call could
stall their latency path.  For them the split-key decode attention keeps its
scratch (the splits' partial outputs, maxima and sums) in a fixed 4 MiB array
inside the library.  This test calls the exported C symbol directly, twice in a
row with different inputs (the array keeps the first call's contents, which must
not leak into the second), and compares each result with the ordinary entry
point that takes caller-provided scratch: both launch the same kernels with the
same splits, so the results must be equal bit for bit.  It also checks that a
call too large for the array is refused, and that a call with one split, which
uses no scratch, is taken at any size.  The ordinary entry point runs first, so
the library (and with it the array, which is part of the loaded module and is
no allocation of any call) is on the device before free memory is compared.
The file sorts last so that a run which stops at the first failure has already
run every other test.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PAGE = 64
SCRATCH_FLOATS = 1 << 20


def _case(nh, nkv, hd, lens, seed):
    g = torch.Generator().manual_seed(seed)
    n_pages = sum((n + PAGE - 1) // PAGE for n in lens) + 2
    kc = torch.randn(n_pages, nkv, PAGE, hd, generator=g).to(torch.bfloat16).to(DEV)
    vc = torch.randn(n_pages, nkv, PAGE, hd, generator=g).to(torch.bfloat16).to(DEV)
    order = torch.randperm(n_pages, generator=g).tolist()
    width = max((n + PAGE - 1) // PAGE for n in lens)
    bt = torch.full((len(lens), width), -1, dtype=torch.int32)
    for s, n in enumerate(lens):
        for i in range((n + PAGE - 1) // PAGE):
            bt[s, i] = order.pop()
    q = torch.randn(len(lens), nh * hd, generator=g).to(torch.bfloat16).to(DEV)
    return q, kc, vc, bt.to(DEV), torch.tensor(lens, dtype=torch.int32, device=DEV)


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


@pytest.mark.parametrize("nh, nkv, hd, n_splits", [(8, 2, 64, 4), (32, 8, 128, 3)])
def test_noalloc_entry_point_matches_the_ordinary_one_twice_in_a_row(nh, nkv, hd, n_splits):
    from janus_b200.kernels import ops
    from janus_b200.kernels.build import ensure_built

    lib = ctypes.CDLL(str(ensure_built("attention_bf16", {"JB_HEAD_DIM": hd})))
    fn = lib.jb_attention_bf16_decode_noalloc
    fn.restype = ctypes.c_int
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    scale = 1.0 / math.sqrt(hd)

    class Scratch:
        def get(self, name, shape, dtype):
            return torch.empty(tuple(shape), dtype=dtype, device=DEV)

    for call, (lens, seed) in enumerate([([700, 130, 5, 64], 1), ([65, 1, 300], 2)]):
        q, kc, vc, bt, kv_len = _case(nh, nkv, hd, lens, seed)
        want = torch.empty_like(q)
        ops.attention_bf16_decode(q, kc, vc, want, bt, kv_len, nh, nkv, hd, PAGE, 0, scale, Scratch(), max(lens),
                                  n_splits=n_splits)
        got = torch.full_like(q, float("nan"))
        free_before = torch.cuda.mem_get_info()[0]
        code = fn(_ptr(q), _ptr(kc), _ptr(vc), _ptr(got), _ptr(bt), _ptr(kv_len), len(lens), nh, nkv, hd, PAGE,
                  bt.shape[1], 0, ctypes.c_float(scale), n_splits, stream)
        torch.cuda.synchronize()
        assert code == 0, f"call {call} returned {code}"
        assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the free device memory"
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got, want), f"call {call}: the two entry points differ"

    # a call that needs more scratch than the array holds is refused, nothing is launched
    n_seqs = SCRATCH_FLOATS // (nh * n_splits * (hd + 2)) + 1
    q, kc, vc, bt, kv_len = _case(nh, nkv, hd, [3] * n_seqs, 3)
    out = torch.zeros_like(q)
    code = fn(_ptr(q), _ptr(kc), _ptr(vc), _ptr(out), _ptr(bt), _ptr(kv_len), n_seqs, nh, nkv, hd, PAGE,
              bt.shape[1], 0, ctypes.c_float(scale), n_splits, stream)
    torch.cuda.synchronize()
    assert code == 10001 and float(out.float().abs().sum()) == 0.0
    # the same batch with one split needs no scratch: it is taken and matches the ordinary entry point
    want = torch.empty_like(q)
    ops.attention_bf16_decode(q, kc, vc, want, bt, kv_len, nh, nkv, hd, PAGE, 0, scale, Scratch(), 3, n_splits=1)
    code = fn(_ptr(q), _ptr(kc), _ptr(vc), _ptr(out), _ptr(bt), _ptr(kv_len), n_seqs, nh, nkv, hd, PAGE,
              bt.shape[1], 0, ctypes.c_float(scale), 1, stream)
    torch.cuda.synchronize()
    assert code == 0 and torch.equal(out, want)
