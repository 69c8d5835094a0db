"""Each CUDA kernel alone against a plain float32/float64 computation of the
same op, at sizes other than the tiny models': widths and vocabularies that are
no power of two, head sizes in steps of 8, any number of heads and groups."""
import math

import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PAGE = 64


@pytest.fixture(scope="module")
def ops():
    from janus_b200.kernels import ops as o
    return o


def close(got, ref, tol):
    got, ref = got.double().cpu(), ref.double().cpu()
    assert torch.isfinite(got).all()
    err = float((got - ref).abs().max() / (ref.abs().max() + 1e-12))
    assert err < tol, f"relative error {err:.3e} >= {tol}"


# ---------------------------------------------------------------- elementwise
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed_gather(ops, dtype):
    V, H, T = 301, 200, 37
    table = torch.randn(V, H, device=DEV).to(dtype)
    ids = torch.randint(0, V, (T,), device=DEV, dtype=torch.int32)
    out = torch.empty(T, H, device=DEV)
    ops.embed_gather(table, ids, out)
    assert torch.equal(out.cpu(), P.embed(table.float().cpu(), ids.cpu()))


@pytest.mark.parametrize("H", [200, 201, 2048, 3000, 4096, 4100, 9000])
@pytest.mark.parametrize("gdt, odt", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16),
                                      (torch.bfloat16, torch.bfloat16)])
def test_rmsnorm(ops, H, gdt, odt):
    """Every build of the kernel: rows of up to 2,048 floats (blocks of 128 threads), of up to 4,096 (256
    threads, four vectors a thread in registers), wider ones (eight vectors, the rest of a row of 9,000 read
    twice), and a width that is no multiple of 4 (scalar loads)."""
    T = 19
    x = torch.randn(T, H, device=DEV) * 3
    gamma = (1 + 0.1 * torch.randn(H, device=DEV)).to(gdt)
    out = torch.empty(T, H, device=DEV, dtype=odt)
    ops.rmsnorm(x, gamma, 1e-6, out)
    ref = P.rms_norm(x.cpu(), gamma.float().cpu(), 1e-6)
    close(out, ref, 2e-6 if odt == torch.float32 else 5e-3)
    rows = torch.tensor([18, 0, 7], device=DEV, dtype=torch.int32)
    out2 = torch.empty(3, H, device=DEV, dtype=odt)
    ops.rmsnorm(x, gamma, 1e-6, out2, rows)
    assert torch.equal(out2, out[rows.long()])


def test_residual_add_and_swiglu(ops):
    T, I = 13, 330
    r = torch.randn(T, I, device=DEV)
    d = torch.randn(T, I, device=DEV).to(torch.bfloat16)
    want = r.cpu() + d.float().cpu()
    ops.residual_add(r, d)
    assert torch.equal(r.cpu(), want)
    gu = torch.randn(T, 2 * I, device=DEV) * 2
    out = torch.empty(T, I, device=DEV)
    ops.swiglu(gu, out)
    close(out, P.silu(gu[:, :I].cpu()) * gu[:, I:].cpu(), 2e-6)


@pytest.mark.parametrize("T, I, up_col, ld", [(13, 328, 384, 768), (5, 131, 256, 512), (64, 8192, 8192, 16384)])
def test_swiglu_of_a_stacked_product(ops, T, I, up_col, ld):
    """The activation kernel behind a gated product that ran as a plain product: float32 rows with the up
    features from a column of their own on, bfloat16 out; four features a thread or one."""
    gu = torch.randn(T, ld, device=DEV) * 2
    out = torch.full((T, I), float("nan"), device=DEV, dtype=torch.bfloat16)
    ops.swiglu_f32_to_bf16(gu, out, up_col)
    ref = (P.silu(gu[:, :I].cpu()) * gu[:, up_col:up_col + I].cpu()).to(torch.bfloat16)
    close(out, ref.float(), 6e-3)


@pytest.mark.parametrize("T", [1, 17, 64])
@pytest.mark.parametrize("I, K", [(192, 64), (320, 96), (1000, 2048)])
def test_gated_product_run_as_plain_product_and_activation(ops, T, I, K):
    """What a narrow layer's gated product does at decode sizes: the packed gated pair read as one stacked
    matrix (gate tiles, then up tiles), a float32 store product, the activation kernel."""
    assert ops.gated_runs_unfused(T, I)
    x, w = bf16_inputs(T, 2 * I, K, T + I + 2)
    w = (w.float() * 3).to(torch.bfloat16)
    gated = ops.pack_gated(w[:I].contiguous(), w[I:].contiguous())
    stacked = gated.stacked()
    gu = torch.full((T, stacked.rows), float("nan"), device=DEV)
    ops.gemm_bf16(x, stacked, gu, mode="store", pair=False)
    y = torch.empty(T, I, device=DEV, dtype=torch.bfloat16)
    ops.swiglu_f32_to_bf16(gu, y, 128 * gated.up_tile_offset)
    ref = P.swiglu_ffn(x.double().cpu(), w[:I].double().cpu(), w[I:].double().cpu(), torch.eye(I, dtype=torch.float64))
    close(y, ref, 6e-3)
    fused = torch.empty(T, I, device=DEV, dtype=torch.bfloat16)
    ops.gemm_bf16(x, gated, fused, mode="swiglu", pair=False)
    close(fused, ref, 6e-3)
    ops.check_kernel_status(torch.device(DEV))


# ---------------------------------------------------------------- rope + cache
@pytest.mark.parametrize("in_dt, out_dt", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16),
                                           (torch.bfloat16, torch.bfloat16)])
def test_rope_cache_write(ops, in_dt, out_dt):
    nh, nkv, hd, T, n_pages = 6, 3, 24, 29, 7
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, device=DEV).to(in_dt)
    positions = torch.randint(0, 300, (T,), device=DEV, dtype=torch.int32)
    dest = torch.randperm(n_pages * PAGE, device=DEV)[:T].to(torch.int32)
    inv = P.rope_inv_freq(hd, 12345.0, None)
    cos, sin = P.rope_cos_sin(torch.arange(300), inv)
    table = torch.stack([cos, sin], -1).contiguous().to(DEV)
    kc = torch.zeros(n_pages, nkv, PAGE, hd, device=DEV, dtype=out_dt)
    vc = torch.zeros_like(kc)
    q = torch.empty(T, nh * hd, device=DEV, dtype=out_dt)
    ops.rope_cache_write(qkv, q, table, positions, dest, kc, vc, nh, nkv, hd, PAGE)
    x = qkv.float().cpu()
    c, s = P.rope_cos_sin(positions.cpu(), inv)
    q_ref = P.apply_rope(x[:, :nh * hd].view(T, nh, hd), c, s).reshape(T, -1)
    k_ref = P.apply_rope(x[:, nh * hd:(nh + nkv) * hd].view(T, nkv, hd), c, s)
    v_ref = x[:, (nh + nkv) * hd:].view(T, nkv, hd)
    tol = 2e-6 if out_dt == torch.float32 else 5e-3
    close(q, q_ref, tol)
    page, row = (dest.cpu() // PAGE).long(), (dest.cpu() % PAGE).long()
    close(kc.cpu()[page, :, row, :], k_ref, tol)
    close(vc.cpu()[page, :, row, :], v_ref, tol)
    untouched = torch.ones(n_pages * PAGE, dtype=torch.bool)
    untouched[dest.cpu().long()] = False
    assert float(kc.cpu().permute(0, 2, 1, 3).reshape(n_pages * PAGE, -1)[untouched].abs().sum()) == 0.0
    # a layer that reads another layer's cache rotates q only
    q2 = torch.empty_like(q)
    ops.rope_cache_write(qkv[:, :nh * hd].contiguous(), q2, table, positions, None, None, None, nh, nkv, hd, PAGE,
                         write_kv=False)
    assert torch.equal(q2, q)


# ---------------------------------------------------------------- float32 product
@pytest.mark.parametrize("T, N, K", [(1, 101, 53), (37, 64, 64), (130, 257, 321),
                                     # up to 16 tokens and rows of whole 16-byte vectors: the weight-streaming kernel
                                     (1, 101, 52), (16, 100, 4100), (9, 300, 64), (17, 70, 128), (64, 40, 200)])
def test_gemm_f32(ops, T, N, K):
    """Both kernels (up to 16 tokens, more) against float64, and a row alone against the same row in its batch,
    bit for bit: the last row alone always takes the small kernel, its batch of more than 16 the other."""
    g = torch.Generator().manual_seed(T + N + K)
    x, w = torch.randn(T, K, generator=g).to(DEV), torch.randn(N, K, generator=g).to(DEV)
    y = torch.empty(T, N, device=DEV)
    ops.gemm_f32(x, w, y)
    ref = x.double().cpu() @ w.double().cpu().T
    # K float32 additions in a row leave a random walk of roundings: about 3.4e-8 sqrt(K) of the largest output
    # (2.2e-6 at K = 4100 on average over seeds, 3.3e-6 at worst of thirty); the bound is four times that
    tol = max(3e-6, 1.5e-7 * math.sqrt(K))
    close(y, ref, tol)
    base = torch.randn(T, N, generator=g).to(DEV)
    y2 = base.clone()
    ops.gemm_f32(x, w, y2, accumulate=True)
    close(y2, ref + base.double().cpu(), tol)
    # a row's result does not depend on the batch it is in
    y1 = torch.empty(1, N, device=DEV)
    ops.gemm_f32(x[T - 1:].contiguous(), w, y1)
    assert torch.equal(y1[0], y[T - 1])


# ---------------------------------------------------------------- paged attention
def paged(k, v, dtype, n_extra_pages=3, seed=0):
    """Scatter dense per-sequence K/V ([len, nkv, hd] each) over shuffled pages.
    Returns (k_cache, v_cache, block_table) with unused entries -1."""
    nkv, hd = k[0].shape[1], k[0].shape[2]
    need = [(x.shape[0] + PAGE - 1) // PAGE for x in k]
    n_pages = sum(need) + n_extra_pages
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(n_pages, generator=g).tolist()
    kc = torch.randn(n_pages, nkv, PAGE, hd, generator=g) * 5      # stale content must never be read
    vc = torch.randn(n_pages, nkv, PAGE, hd, generator=g) * 5
    bt = torch.full((len(k), max(need)), -1, dtype=torch.int32)
    for s, (ks, vs) in enumerate(zip(k, v)):
        for i in range(need[s]):
            p = perm.pop()
            bt[s, i] = p
            n = min(PAGE, ks.shape[0] - i * PAGE)
            kc[p, :, :n] = ks[i * PAGE:i * PAGE + n].transpose(0, 1)
            vc[p, :, :n] = vs[i * PAGE:i * PAGE + n].transpose(0, 1)
    return kc.to(DEV).to(dtype), vc.to(DEV).to(dtype), bt.to(DEV)


def attention_case(nh, nkv, hd, lens, q_lens, dtype, seed=0, spike=True):
    """Sequences of `lens` keys whose last `q_lens` tokens are the queries."""
    g = torch.Generator().manual_seed(seed)
    rnd = lambda *s: torch.randn(*s, generator=g).to(dtype).float()   # values exactly representable in `dtype`
    qs, ks, vs = [], [], []
    for n, nq in zip(lens, q_lens):
        q, k, v = rnd(n, nh, hd), rnd(n, nkv, hd), rnd(n, nkv, hd)
        if spike and n > 3:
            # one far key stands out for the last query: a kernel that misses it is far off
            k[1] = (q[n - 1, 0] * 1.5).to(dtype).float()
            v[1] = (v[1] + 3.0).to(dtype).float()
        qs.append(q); ks.append(k); vs.append(v)
    return qs, ks, vs


def plain_attention_rows(qs, ks, vs, q_lens, window):
    outs = []
    for q, k, v, nq in zip(qs, ks, vs, q_lens):
        full = P.attention(q, k, v, window=window if window > 0 else None)
        outs.append(full[q.shape[0] - nq:].reshape(nq, -1))
    return torch.cat(outs, 0)


@pytest.mark.parametrize("nh, nkv, hd, window", [(4, 2, 16, 0), (6, 2, 24, 0), (3, 1, 40, 0), (5, 5, 72, 70),
                                                 (8, 2, 256, 0)])
def test_attention_f32(ops, nh, nkv, hd, window):
    lens, q_lens = [130, 5, 64, 200], [130, 1, 3, 17]
    qs, ks, vs = attention_case(nh, nkv, hd, lens, q_lens, torch.float32)
    kc, vc, bt = paged(ks, vs, torch.float32)
    q = torch.cat([x[n - nq:].reshape(nq, -1) for x, n, nq in zip(qs, lens, q_lens)]).to(DEV)
    token_seq = torch.cat([torch.full((nq,), i) for i, nq in enumerate(q_lens)]).to(DEV).int()
    positions = torch.cat([torch.arange(n - nq, n) for n, nq in zip(lens, q_lens)]).to(DEV).int()
    out = torch.empty_like(q)
    ops.attention_f32(q, kc, vc, out, bt, token_seq, positions, nh, nkv, hd, PAGE, window, 1 / math.sqrt(hd))
    close(out, plain_attention_rows(qs, ks, vs, q_lens, window), 2e-5)


@pytest.mark.parametrize("nh, nkv, hd, window", [(4, 2, 16, 0), (6, 2, 24, 0), (3, 1, 40, 0), (5, 5, 72, 70),
                                                 (32, 8, 128, 0), (8, 1, 64, 100), (40, 2, 32, 0), (4, 4, 256, 0)])
def test_attention_bf16_prefill(ops, nh, nkv, hd, window):
    lens, q_lens = [130, 5, 64, 200, 1], [130, 2, 64, 17, 1]
    qs, ks, vs = attention_case(nh, nkv, hd, lens, q_lens, torch.bfloat16)
    kc, vc, bt = paged(ks, vs, torch.bfloat16)
    q = torch.cat([x[n - nq:].reshape(nq, -1) for x, n, nq in zip(qs, lens, q_lens)]).to(DEV).to(torch.bfloat16)
    q_start = torch.tensor([0] + torch.tensor(q_lens).cumsum(0).tolist(), device=DEV, dtype=torch.int32)
    kv_len = torch.tensor(lens, device=DEV, dtype=torch.int32)
    out = torch.empty_like(q)
    ops.attention_bf16_prefill(q, kc, vc, out, bt, q_start, kv_len, len(lens), max(q_lens), nh, nkv, hd, PAGE,
                               window, 1 / math.sqrt(hd))
    close(out, plain_attention_rows(qs, ks, vs, q_lens, window), 1.5e-2)


@pytest.mark.parametrize("tiles", ["1", "2"])
@pytest.mark.parametrize("nh, nkv, hd, window", [(32, 8, 128, 0), (8, 1, 64, 100), (4, 4, 128, 0), (16, 2, 128, 70),
                                                 (2, 1, 64, 0), (64, 1, 128, 0),
                                                 # groups that do not divide the 128 rows of a tile: 3, 5, 6, 7, 100
                                                 (24, 8, 128, 0), (10, 2, 128, 90), (6, 1, 64, 50), (12, 4, 64, 0),
                                                 (7, 1, 128, 0), (100, 1, 64, 0),
                                                 # head sizes that fill a row of 64 or 128 dims only in part: the
                                                 # rest arrives as zeros, a last 16-dim step or store may be half
                                                 (6, 2, 96, 0), (4, 1, 40, 70), (8, 8, 80, 0), (5, 1, 120, 0),
                                                 (9, 3, 24, 0), (4, 2, 8, 0), (12, 4, 104, 90), (8, 2, 56, 0),
                                                 (16, 4, 112, 0), (4, 4, 72, 0), (3, 1, 48, 30),
                                                 # rows of 256 dims: the one-tile kernel with a ring of two pages
                                                 (4, 2, 256, 0), (6, 2, 192, 100), (5, 1, 136, 0), (8, 8, 200, 0),
                                                 (3, 3, 248, 70)])
def test_attention_tc_prefill(ops, nh, nkv, hd, window, tiles, monkeypatch):
    """The tcgen05 kernel against the plain attention: ragged batch, chunked prompts
    (queries are the last q_len positions), a far key that stands out; the one-tile kernel and the
    two-tile kernel over blocks of 128 keys.
    With a window the first page of a tile holds a few keys for some warps and none for the others, so
    warps of one CTA run far apart: repeated, since a wait that mistakes one block's completion for
    another's shows only now and then."""
    assert ops.attention_tc_supported(nh, nkv, hd)
    monkeypatch.setenv("JANUS_ATTN_TC_TILES", tiles)
    lens, q_lens = [130, 5, 64, 300, 1, 257], [130, 2, 64, 17, 1, 257]
    qs, ks, vs = attention_case(nh, nkv, hd, lens, q_lens, torch.bfloat16, seed=3)
    kc, vc, bt = paged(ks, vs, torch.bfloat16, seed=3)
    q = torch.cat([x[n - nq:].reshape(nq, -1) for x, n, nq in zip(qs, lens, q_lens)]).to(DEV).to(torch.bfloat16)
    q_start = torch.tensor([0] + torch.tensor(q_lens).cumsum(0).tolist(), device=DEV, dtype=torch.int32)
    kv_len = torch.tensor(lens, device=DEV, dtype=torch.int32)
    ref = plain_attention_rows(qs, ks, vs, q_lens, window)
    for _ in range(4 if window else 1):
        out = torch.full_like(q, float("nan"))
        ops.attention_tc_prefill(q, kc, vc, out, bt, q_start, kv_len, len(lens), max(q_lens), nh, nkv, hd, PAGE,
                                 window, 1 / math.sqrt(hd))
        ops.check_kernel_status(torch.device(DEV))
        close(out, ref, 1.5e-2)


@pytest.mark.parametrize("tiles", ["1", "2"])
@pytest.mark.parametrize("nh, nkv, hd, window", [(32, 8, 128, 0), (6, 2, 96, 90), (8, 1, 64, 0)])
def test_attention_tc_prefill_head_after_head(ops, nh, nkv, hd, window, tiles, monkeypatch):
    """A block table wide enough for sequences whose keys and values would overflow L2 makes the kernel hand
    its CTAs out head after head instead of kv heads fastest (the grid's x and y change places): the same
    results."""
    monkeypatch.setenv("JANUS_ATTN_TC_TILES", tiles)
    lens, q_lens = [130, 5, 300, 257], [130, 2, 17, 257]
    qs, ks, vs = attention_case(nh, nkv, hd, lens, q_lens, torch.bfloat16, seed=4)
    kc, vc, bt = paged(ks, vs, torch.bfloat16, seed=4)
    width = 96 * 1024 * 1024 // (PAGE * nkv * hd * 4) + 8
    bt = torch.cat([bt, torch.full((bt.shape[0], width), -1, dtype=bt.dtype, device=bt.device)], 1).contiguous()
    q = torch.cat([x[n - nq:].reshape(nq, -1) for x, n, nq in zip(qs, lens, q_lens)]).to(DEV).to(torch.bfloat16)
    q_start = torch.tensor([0] + torch.tensor(q_lens).cumsum(0).tolist(), device=DEV, dtype=torch.int32)
    kv_len = torch.tensor(lens, device=DEV, dtype=torch.int32)
    out = torch.full_like(q, float("nan"))
    ops.attention_tc_prefill(q, kc, vc, out, bt, q_start, kv_len, len(lens), max(q_lens), nh, nkv, hd, PAGE,
                             window, 1 / math.sqrt(hd))
    ops.check_kernel_status(torch.device(DEV))
    close(out, plain_attention_rows(qs, ks, vs, q_lens, window), 1.5e-2)


class _WS:
    def __init__(self):
        self.bufs = {}

    def get(self, name, shape, dtype):
        self.bufs[name] = torch.full(tuple(shape), float("nan"), device=DEV, dtype=dtype)
        return self.bufs[name]


@pytest.mark.parametrize("nh, nkv, hd, window", [(4, 2, 16, 0), (3, 1, 40, 0), (32, 8, 128, 0), (5, 5, 72, 70),
                                                 (40, 2, 32, 0), (4, 4, 256, 0)])
@pytest.mark.parametrize("n_splits", [1, 3, None, 8, 16, 20])
def test_attention_bf16_decode(ops, nh, nkv, hd, window, n_splits):
    """One split writes the result itself, more meet in scratch and a joining kernel; a sequence of one key
    leaves most of 8 to 20 splits without a page."""
    lens = [130, 5, 64, 1, 700, 65]
    q_lens = [1] * len(lens)
    qs, ks, vs = attention_case(nh, nkv, hd, lens, q_lens, torch.bfloat16, seed=1)
    kc, vc, bt = paged(ks, vs, torch.bfloat16, seed=1)
    q = torch.cat([x[n - 1:].reshape(1, -1) for x, n in zip(qs, lens)]).to(DEV).to(torch.bfloat16)
    kv_len = torch.tensor(lens, device=DEV, dtype=torch.int32)
    out = torch.empty_like(q)
    ops.attention_bf16_decode(q, kc, vc, out, bt, kv_len, nh, nkv, hd, PAGE, window, 1 / math.sqrt(hd), _WS(),
                              max(lens), n_splits=n_splits)
    close(out, plain_attention_rows(qs, ks, vs, q_lens, window), 1.5e-2)


def _last_rows_attention(q, k, v, nq, window):
    """Plain attention of the last `nq` positions of one sequence (q [n, nh, hd], k, v [n, nkv, hd]) in float64:
    row i sees keys up to its own position, from `window` keys back."""
    n, nh, hd = q.shape
    nkv = k.shape[1]
    qq = q[n - nq:].double()
    kk = k.double().repeat_interleave(nh // nkv, 1)
    vv = v.double().repeat_interleave(nh // nkv, 1)
    scores = torch.einsum("qhd,khd->hqk", qq, kk) / math.sqrt(hd)
    pos = torch.arange(n - nq, n)[:, None]
    key = torch.arange(n)[None, :]
    seen = (key <= pos) & ((key > pos - window) if window > 0 else torch.ones_like(key, dtype=torch.bool))
    scores = scores.masked_fill(~seen[None], float("-inf"))
    return torch.einsum("hqk,khd->qhd", torch.softmax(scores, -1), vv).reshape(nq, nh * hd).float()


@pytest.mark.parametrize("window", [0, 50000])
def test_attention_over_a_context_of_70000_keys(ops, window):
    """Far beyond the engine tests' lengths: 1,094 pages a sequence, a key near the start that stands out for the
    last query (a kernel that loses count of its pages or splits is far off), one token decoded (splits chosen by
    the library and 32 given) and the last 70 tokens of the sequence as a prompt chunk on both prompt kernels;
    with a window of 50,000 the standing-out key lies outside and must not count."""
    nh, nkv, hd, n, nq = 4, 1, 128, 70000, 70
    qs, ks, vs = attention_case(nh, nkv, hd, [n], [nq], torch.bfloat16, seed=6)
    kc, vc, bt = paged(ks, vs, torch.bfloat16, seed=6)
    ref = _last_rows_attention(qs[0], ks[0], vs[0], nq, window)
    scale = 1 / math.sqrt(hd)
    kv_len = torch.tensor([n], device=DEV, dtype=torch.int32)
    q1 = qs[0][n - 1:].reshape(1, -1).to(DEV).to(torch.bfloat16)
    for n_splits in (None, 32):
        out = torch.full_like(q1, float("nan"))
        ops.attention_bf16_decode(q1, kc, vc, out, bt, kv_len, nh, nkv, hd, PAGE, window, scale, _WS(), n,
                                  n_splits=n_splits)
        close(out, ref[-1:], 1.5e-2)
    q = qs[0][n - nq:].reshape(nq, -1).to(DEV).to(torch.bfloat16)
    q_start = torch.tensor([0, nq], device=DEV, dtype=torch.int32)
    for face in (ops.attention_tc_prefill, ops.attention_bf16_prefill):
        out = torch.full_like(q, float("nan"))
        face(q, kc, vc, out, bt, q_start, kv_len, 1, nq, nh, nkv, hd, PAGE, window, scale)
        ops.check_kernel_status(torch.device(DEV))
        close(out, ref, 1.5e-2)


@pytest.mark.parametrize("nh, nkv, hd, window, rotate", [(4, 2, 16, 0, True), (3, 1, 40, 0, True), (32, 8, 128, 0, True),
                                                         (5, 5, 72, 70, False), (40, 2, 32, 0, True)])
def test_attention_bf16_decode_with_fused_rotation_and_append(ops, nh, nkv, hd, window, rotate):
    """The decode kernel fed with the projection's float32 q/k/v (it rotates, appends to the cache
    and attends) against the two-kernel path: rotate + append, then attend."""
    lens = [130, 5, 64, 1, 700, 65, 128]
    B = len(lens)
    _, ks, vs = attention_case(nh, nkv, hd, lens, [1] * B, torch.bfloat16, seed=2, spike=False)
    kc, vc, bt = paged(ks, vs, torch.bfloat16, seed=2)
    g = torch.Generator().manual_seed(5)
    qkv = torch.randn(B, (nh + 2 * nkv) * hd, generator=g).to(DEV)
    kv_len = torch.tensor(lens, device=DEV, dtype=torch.int32)
    positions = kv_len - 1
    dest = torch.stack([bt[i, (n - 1) // PAGE] * PAGE + (n - 1) % PAGE for i, n in enumerate(lens)]).to(torch.int32)
    table = None
    if rotate:
        cos, sin = P.rope_cos_sin(torch.arange(800), P.rope_inv_freq(hd, 10000.0, None))
        table = torch.stack([cos, sin], -1).contiguous().to(DEV)
    scale = 1 / math.sqrt(hd)
    for n_splits in (1, 3):
        k1, v1, k2, v2 = kc.clone(), vc.clone(), kc.clone(), vc.clone()
        q = torch.empty(B, nh * hd, device=DEV, dtype=torch.bfloat16)
        ops.rope_cache_write(qkv, q, table, positions, dest, k1, v1, nh, nkv, hd, PAGE)
        want = torch.empty_like(q)
        ops.attention_bf16_decode(q, k1, v1, want, bt, kv_len, nh, nkv, hd, PAGE, window, scale, _WS(), max(lens),
                                  n_splits=n_splits)
        got = torch.full_like(q, float("nan"))
        ops.attention_bf16_decode(None, k2, v2, got, bt, kv_len, nh, nkv, hd, PAGE, window, scale, _WS(), max(lens),
                                  n_splits=n_splits, qkv=qkv, cos_sin=table, dest=dest)
        assert torch.equal(k1, k2) and torch.equal(v1, v2)          # the same rows were appended
        close(got, want.float(), 4e-3)


# ---------------------------------------------------------------- tensor-core product
def bf16_inputs(T, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    return x.to(DEV), w.to(DEV)


@pytest.mark.parametrize("T", [1, 5, 16, 33, 64, 100, 300])
@pytest.mark.parametrize("N, K", [(200, 120), (128, 64), (1000, 320), (384, 4096)])
def test_gemm_bf16_store_and_add(ops, T, N, K):
    x, w = bf16_inputs(T, N, K, T + N)
    ref = x.double().cpu() @ w.double().cpu().T
    w = ops.pack_weight(w)
    y16 = torch.empty(T, N, device=DEV, dtype=torch.bfloat16)
    ops.gemm_bf16(x, w, y16, pair=False)
    close(y16, ref, 6e-3)
    y32 = torch.full((T, N), float("nan"), device=DEV)
    ops.gemm_bf16(x, w, y32, pair=False)
    close(y32, ref, 2e-5)
    base = torch.randn(T, N, device=DEV)
    for split in (1, None, 4):
        acc = base.clone()
        ops.gemm_bf16(x, w, acc, mode="add", split_k=split, pair=False)
        close(acc, ref + base.double().cpu(), 2e-5)
    acc = base.clone()
    ops.gemm_bf16(x, w, acc, mode="add")          # kernel and slices of K as the cost estimate picks them
    close(acc, ref + base.double().cpu(), 2e-5)
    ops.check_kernel_status(torch.device(DEV))


@pytest.mark.parametrize("T", [1, 5, 16, 33, 64, 100, 300])
@pytest.mark.parametrize("N, K", [(200, 1024), (1000, 640), (384, 4096)])
def test_gemm_bf16_slices_summed_in_order(ops, T, N, K):
    """Deterministic mode: every slice of K leaves its tile in scratch and the slice that arrives last sums them
    in slice order.  Right against the plain product, and the same bits when run again (atomic adds are not)."""
    x, w = bf16_inputs(T, N, K, T + N + 3)
    ref = x.double().cpu() @ w.double().cpu().T
    w = ops.pack_weight(w)
    base = torch.randn(T, N, device=DEV)
    ops.set_deterministic(True)
    try:
        for split in (2, 3, 7, 1000):
            got = []
            for _ in range(3):
                acc = base.clone()
                ops.gemm_bf16(x, w, acc, mode="add", split_k=split, pair=False)
                got.append(acc)
            close(got[0], ref + base.double().cpu(), 2e-5)
            assert torch.equal(got[0], got[1]) and torch.equal(got[0], got[2])
        acc = base.clone()
        ops.gemm_bf16(x, w, acc, mode="add")              # as the plan picks kernel and slices
        close(acc, ref + base.double().cpu(), 2e-5)
    finally:
        ops.set_deterministic(False)
    ops.check_kernel_status(torch.device(DEV))


@pytest.mark.parametrize("T", [1, 17, 64, 200])
@pytest.mark.parametrize("I, K", [(192, 64), (320, 96), (1000, 2048)])
def test_gemm_bf16_swiglu(ops, T, I, K):
    x, w = bf16_inputs(T, 2 * I, K, T + I)
    w = (w.float() * 3).to(torch.bfloat16)
    y = torch.empty(T, I, device=DEV, dtype=torch.bfloat16)
    ops.gemm_bf16(x, ops.pack_gated(w[:I].contiguous(), w[I:].contiguous()), y, mode="swiglu", pair=False)
    ref = P.swiglu_ffn(x.double().cpu(), w[:I].double().cpu(), w[I:].double().cpu(), torch.eye(I, dtype=torch.float64))
    close(y, ref, 6e-3)
    ops.check_kernel_status(torch.device(DEV))


@pytest.mark.parametrize("T", [70, 130, 256, 300, 513, 1100])
@pytest.mark.parametrize("N, K", [(200, 120), (256, 64), (1000, 320), (640, 4096), (4096, 1096)])
def test_gemm_bf16_cta_pairs(ops, T, N, K):
    """The cta_group::2 kernel (256 weight rows per CTA pair, each CTA loads half of the token tile):
    ragged token counts, widths that are no multiple of 256, a K tail, several tiles per pair."""
    x, w = bf16_inputs(T, N, K, T + N + 1)
    ref = x.double().cpu() @ w.double().cpu().T
    w = ops.pack_weight(w)
    y16 = torch.empty(T, N, device=DEV, dtype=torch.bfloat16)
    ops.gemm_bf16(x, w, y16, pair=True)
    close(y16, ref, 6e-3)
    y32 = torch.full((T, N), float("nan"), device=DEV)
    ops.gemm_bf16(x, w, y32, pair=True)
    close(y32, ref, 2e-5)
    base = torch.randn(T, N, device=DEV)
    acc = base.clone()
    ops.gemm_bf16(x, w, acc, mode="add", pair=True)
    close(acc, ref + base.double().cpu(), 2e-5)
    for split in (2, 5, 1000):                    # slices of K meet by atomic adds; never more slices than k-tiles
        acc = base.clone()
        ops.gemm_bf16(x, w, acc, mode="add", pair=True, split_k=split)
        close(acc, ref + base.double().cpu(), 2e-5)
    tiles = ((T + 255) // 256) * ((N + 255) // 256)
    for whole in sorted({1, tiles // 2, tiles - 1, tiles, tiles + 5} - {0}):   # the first tiles whole, the others in slices
        acc = base.clone()
        ops.gemm_bf16(x, w, acc, mode="add", pair=True, split_k=3, whole_tiles=whole)
        close(acc, ref + base.double().cpu(), 2e-5)
    ops.check_kernel_status(torch.device(DEV))


@pytest.mark.parametrize("T, N, K", [(2500, 200, 120), (2500, 1000, 320), (4400, 700, 64), (2049, 520, 96)])
def test_gemm_bf16_cta_pairs_beyond_one_band_of_token_tiles(ops, T, N, K):
    """More than eight token tiles: output tiles are numbered in bands of eight token tiles, the last band holds
    fewer (2,500 tokens: 8 + 2 tiles; 4,400: 8 + 8 + 2; 2,049: 8 + 1).  Every tile is computed once, whole or in
    slices, whichever of them are the uncut ones."""
    x, w = bf16_inputs(T, N, K, T + N + 1)
    ref = x.double().cpu() @ w.double().cpu().T
    w = ops.pack_weight(w)
    y32 = torch.full((T, N), float("nan"), device=DEV)
    ops.gemm_bf16(x, w, y32, pair=True)
    close(y32, ref, 2e-5)
    base = torch.randn(T, N, device=DEV)
    tiles = ((T + 255) // 256) * ((N + 255) // 256)
    for split, whole in ((1, 0), (2, 0), (3, 5), (3, tiles - 3), (2, 17)):
        acc = base.clone()
        ops.gemm_bf16(x, w, acc, mode="add", pair=True, split_k=split, whole_tiles=whole)
        close(acc, ref + base.double().cpu(), 2e-5)
    ops.check_kernel_status(torch.device(DEV))


@pytest.mark.parametrize("T", [70, 130, 256, 700, 2500])
@pytest.mark.parametrize("I, K", [(192, 64), (320, 96), (1000, 2048)])
def test_gemm_bf16_cta_pairs_swiglu(ops, T, I, K):
    x, w = bf16_inputs(T, 2 * I, K, T + I + 1)
    w = (w.float() * 3).to(torch.bfloat16)
    y = torch.empty(T, I, device=DEV, dtype=torch.bfloat16)
    ops.gemm_bf16(x, ops.pack_gated(w[:I].contiguous(), w[I:].contiguous()), y, mode="swiglu", pair=True)
    ref = P.swiglu_ffn(x.double().cpu(), w[:I].double().cpu(), w[I:].double().cpu(), torch.eye(I, dtype=torch.float64))
    close(y, ref, 6e-3)
    ops.check_kernel_status(torch.device(DEV))


@pytest.mark.parametrize("T", [256, 700, 2500])
@pytest.mark.parametrize("nh, nkv, hd, K", [(3, 1, 128, 320), (6, 3, 64, 96), (5, 5, 32, 2048), (2, 1, 256, 64)])
def test_gemm_qkv_with_rotation_and_cache_append(ops, T, nh, nkv, hd, K):
    """The stacked q/k/v projection whose epilogue rotates q and k and writes k, v into the paged cache:
    widths that are no multiple of the 256-column tile, tiles that hold q, k and v heads side by side."""
    n_pages = (T + PAGE - 1) // PAGE + 3
    x, w = bf16_inputs(T, (nh + 2 * nkv) * hd, K, T + hd)
    positions = torch.randint(0, 900, (T,), device=DEV, dtype=torch.int32)
    dest = torch.randperm(n_pages * PAGE, device=DEV)[:T].to(torch.int32)
    inv = P.rope_inv_freq(hd, 50000.0, None)
    cos, sin = P.rope_cos_sin(torch.arange(900), inv)
    table = torch.stack([cos, sin], -1).contiguous().to(DEV)
    kc = torch.zeros(n_pages, nkv, PAGE, hd, device=DEV, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    q = torch.full((T, nh * hd), float("nan"), device=DEV, dtype=torch.bfloat16)
    ops.gemm_qkv_rope_cache(x, ops.pack_weight(w), q, table, positions, dest, kc, vc, nh, nkv, hd, PAGE)
    ops.check_kernel_status(torch.device(DEV))
    y = x.double().cpu() @ w.double().cpu().T
    c, s_ = P.rope_cos_sin(positions.cpu(), inv)
    q_ref = P.apply_rope(y[:, :nh * hd].view(T, nh, hd), c.double(), s_.double()).reshape(T, -1)
    k_ref = P.apply_rope(y[:, nh * hd:(nh + nkv) * hd].view(T, nkv, hd), c.double(), s_.double())
    v_ref = y[:, (nh + nkv) * hd:].view(T, nkv, hd)
    close(q, q_ref, 6e-3)
    page, row = (dest.cpu() // PAGE).long(), (dest.cpu() % PAGE).long()
    close(kc.cpu()[page, :, row, :], k_ref, 6e-3)
    close(vc.cpu()[page, :, row, :], v_ref, 6e-3)
    untouched = torch.ones(n_pages * PAGE, dtype=torch.bool)
    untouched[dest.cpu().long()] = False
    for cache in (kc, vc):
        assert float(cache.float().cpu().permute(0, 2, 1, 3).reshape(n_pages * PAGE, -1)[untouched].abs().sum()) == 0.0


def _guarded(shape, dtype, fill):
    """A tensor in the middle of a larger buffer whose rest holds a guard value."""
    n = math.prod(shape)
    pad = 4096
    buf = torch.full((n + 2 * pad,), fill, device=DEV, dtype=dtype)
    return buf, buf[pad:pad + n].view(*shape), pad


def _guards_intact(buf, pad, fill):
    head, tail = buf[:pad].float().cpu(), buf[-pad:].float().cpu()
    return bool((head == fill).all()) and bool((tail == fill).all())


@pytest.mark.parametrize("T", [5, 33, 300, 700])
def test_kernels_write_nothing_outside_their_outputs(ops, T):
    """Guard values before and after every output of the bfloat16 path stay as they were, at token counts and
    widths that leave the last tile of every kernel partly empty."""
    N, K, I, nh, nkv, hd = 200, 120, 104, 5, 5, 40
    x, w = bf16_inputs(T, N, K, T)
    w = ops.pack_weight(w)
    for dtype, mode in ((torch.bfloat16, "store"), (torch.float32, "store"), (torch.float32, "add")):
        buf, y, pad = _guarded((T, N), dtype, 7.0)
        ops.gemm_bf16(x, w, y, mode=mode)
        assert _guards_intact(buf, pad, 7.0), (T, dtype, mode)
    _, wg = bf16_inputs(T, 2 * I, K, T + 1)
    wg = ops.pack_gated(wg[:I].contiguous(), wg[I:].contiguous())
    buf, act, pad = _guarded((T, I), torch.bfloat16, 7.0)
    ops.gemm_bf16(x, wg, act, mode="swiglu")
    assert _guards_intact(buf, pad, 7.0)
    if T >= 256:                                        # the CTA-pair kernels, asked for by name
        for dtype, mode in ((torch.float32, "store"), (torch.float32, "add")):
            buf, y, pad = _guarded((T, N), dtype, 7.0)
            ops.gemm_bf16(x, w, y, mode=mode, pair=True)
            assert _guards_intact(buf, pad, 7.0), (T, dtype, mode)
        buf, act, pad = _guarded((T, I), torch.bfloat16, 7.0)
        ops.gemm_bf16(x, wg, act, mode="swiglu", pair=True)
        assert _guards_intact(buf, pad, 7.0)
    # norm and the rotation with cache append
    res = torch.randn(T, K, device=DEV)
    gamma = torch.ones(K, device=DEV, dtype=torch.bfloat16)
    buf, normed, pad = _guarded((T, K), torch.bfloat16, 7.0)
    ops.rmsnorm(res, gamma, 1e-5, normed)
    assert _guards_intact(buf, pad, 7.0)
    n_pages = (T + PAGE - 1) // PAGE
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, device=DEV)
    cos, sin = P.rope_cos_sin(torch.arange(T), P.rope_inv_freq(hd, 10000.0, None))
    table = torch.stack([cos, sin], -1).contiguous().to(DEV)
    positions = torch.arange(T, device=DEV, dtype=torch.int32)
    bq, q, pq = _guarded((T, nh * hd), torch.bfloat16, 7.0)
    bk, kc, pk = _guarded((n_pages, nkv, PAGE, hd), torch.bfloat16, 7.0)
    bv, vc, pv = _guarded((n_pages, nkv, PAGE, hd), torch.bfloat16, 7.0)
    ops.rope_cache_write(qkv, q, table, positions, positions, kc, vc, nh, nkv, hd, PAGE)
    assert _guards_intact(bq, pq, 7.0) and _guards_intact(bk, pk, 7.0) and _guards_intact(bv, pv, 7.0)
    # attention of the last token of one sequence of T keys over those pages, and of the whole prompt
    table_pages = torch.arange(n_pages, device=DEV, dtype=torch.int32).view(1, n_pages)
    kv_len = torch.tensor([T], device=DEV, dtype=torch.int32)
    bo, out, po = _guarded((1, nh * hd), torch.bfloat16, 7.0)
    ops.attention_bf16_decode(q[T - 1:].contiguous(), kc, vc, out, table_pages, kv_len, nh, nkv, hd, PAGE, 0,
                              1 / math.sqrt(hd), _WS(), T, n_splits=3)
    assert _guards_intact(bo, po, 7.0)
    q_start = torch.tensor([0, T], device=DEV, dtype=torch.int32)
    bo, out, po = _guarded((T, nh * hd), torch.bfloat16, 7.0)
    ops.attention_bf16_prefill(q, kc, vc, out, table_pages, q_start, kv_len, 1, T, nh, nkv, hd, PAGE, 0, 1 / math.sqrt(hd))
    assert _guards_intact(bo, po, 7.0)
    ops.check_kernel_status(torch.device(DEV))


def test_a_wait_that_runs_out_is_reported_and_the_device_stays_usable(ops, monkeypatch):
    """Every wait of the tensor-core kernels on an mbarrier has a time limit.  A build for this test alone has
    a limit of 3 ms and a producer warp that asks for no tile at all, so nothing is in flight: the MMA warp's
    and the epilogue's waits run out, the kernel records who gave up, frees its TMEM and returns.  The host
    reads the status word as a `KernelError`, the word is cleared, and an ordinary product afterwards is right."""
    dev = torch.device(DEV)
    ops.check_kernel_status(dev)
    x, w = bf16_inputs(8, 128, 64, 3)
    packed = ops.pack_weight(w)
    y = torch.zeros(8, 128, device=DEV)
    monkeypatch.setattr(ops, "_GEMM_DEFINES", {"JB_WAIT_LIMIT_NS": 3000000, "JB_TEST_NO_LOADS": 1})
    ops.gemm_bf16(x, packed, y, mode="store", pair=False)          # one tile, one CTA; returns after about 6 ms
    with pytest.raises(ops.KernelError, match="timed out waiting on an mbarrier"):
        ops.check_kernel_status(dev)
    monkeypatch.undo()
    ops.check_kernel_status(dev)                                    # the word was cleared
    assert int(ops.kernel_status(dev).item()) == 0
    ops.gemm_bf16(x, packed, y, mode="store", pair=False)
    close(y, x.double().cpu() @ w.double().cpu().T, 2e-5)
    ops.check_kernel_status(dev)


def test_gemm_bf16_refuses_what_it_cannot_take(ops):
    w = torch.zeros(16, 100, device=DEV, dtype=torch.bfloat16)       # K = 100 is not a multiple of 8
    with pytest.raises(Exception, match="multiple of 8"):
        ops.pack_weight(w)
    x = torch.zeros(4, 104, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(Exception, match="packed"):                    # a row-major matrix is no weight of a product
        ops.gemm_bf16(x, torch.zeros(16, 104, device=DEV, dtype=torch.bfloat16),
                      torch.empty(4, 16, device=DEV, dtype=torch.bfloat16))
    with pytest.raises(Exception, match="does not fit"):
        ops.gemm_bf16(x, ops.pack_weight(torch.zeros(16, 96, device=DEV, dtype=torch.bfloat16)),
                      torch.empty(4, 16, device=DEV, dtype=torch.bfloat16))


@pytest.mark.parametrize("N, K", [(1, 8), (200, 120), (128, 64), (300, 4096)])
def test_pack_weight_layout(ops, N, K):
    """Tiles of 128 x 64, zero-padded, [row tile][k tile]; chunk c (8 values) of row r at chunk c ^ (r & 7)."""
    w = torch.randn(N, K, device=DEV).to(torch.bfloat16)
    packed = ops.pack_weight(w)
    rt, kt = (N + 127) // 128, (K + 63) // 64
    assert tuple(packed.tiles.shape) == (rt, kt, 128, 64) and (packed.rows, packed.cols) == (N, K)
    padded = torch.zeros(rt * 128, kt * 64, dtype=torch.bfloat16)
    padded[:N, :K] = w.cpu()
    tiles = padded.view(rt, 128, kt, 8, 8).permute(0, 2, 1, 3, 4)            # [rt, kt, row, chunk, 8]
    r = torch.arange(128) & 7
    src = torch.arange(8)[None, :] ^ r[:, None]                               # chunk stored at position p
    want = torch.gather(tiles, 3, src[None, None, :, :, None].expand(rt, kt, 128, 8, 8)).reshape(rt, kt, 128, 64)
    assert torch.equal(packed.tiles.cpu(), want)
    sub = packed.first_rows(min(N, 130))
    assert sub.tiles.data_ptr() == packed.tiles.data_ptr() and sub.rows == min(N, 130)


# ---------------------------------------------------------------- sampling
def run_sample(ops, logits, temperature, top_k=0, top_p=1.0, penalty=1.0, counts=None, seed=11, steps=None):
    B, V = logits.shape
    out = torch.empty(B, dtype=torch.int32, device=DEV)
    seq = torch.arange(B, dtype=torch.int32, device=DEV)
    st = torch.zeros(B, dtype=torch.int32, device=DEV) if steps is None else steps
    rows = torch.arange(B, dtype=torch.int32, device=DEV)
    ops.sample(logits, out, temperature, top_k, top_p, penalty, counts, rows, seed, seq, st)
    return out.cpu().tolist()


def test_greedy_lowest_index_wins(ops):
    V = 1000
    logits = torch.randn(5, V, device=DEV)
    logits[0, 700] = logits[0, 300] = 50.0
    logits[1, V - 1] = 60.0
    logits[2, 0] = 60.0
    got = run_sample(ops, logits, 0.0)
    assert got == [P.argmax_lowest(logits[i].cpu()) for i in range(5)] and got[:3] == [300, V - 1, 0]


def test_the_reference_s_own_sampler_cases_on_the_device(ops):
    """The vectors of the reference's sampler tests (crates/janus-engine/src/model/sampler.rs:871-891, 955-1000)
    through the sampling kernel: the greedy pick, a NaN among the logits (it never wins), and the batch of two
    rows with the default repetition penalty of 1.15 over contexts [1, 2] and [5, 6]."""
    for logits, want in (([0.1, 0.5, 0.3, 0.9, 0.2], 3), ([5.0, 1.0, 3.0], 0), ([-1.0, -5.0, -0.5], 2),
                         ([0.1, float("nan"), 0.3, 0.2], 2)):
        assert run_sample(ops, torch.tensor([logits], device=DEV), 0.0) == [want]
    rows = torch.tensor([[0.1, 0.2, 0.3, 0.9, 0.4, 0.1, 0.2, 0.1, 0.3, 0.2],
                         [0.2, 0.1, 0.3, 0.2, 0.1, 0.4, 0.3, 0.8, 0.2, 0.1]], device=DEV)
    counts = torch.zeros(2, 10, dtype=torch.int32, device=DEV)
    counts[0, 1] = counts[0, 2] = counts[1, 5] = counts[1, 6] = 1
    assert run_sample(ops, rows, 0.0, penalty=1.15, counts=counts) == [3, 7]
    # crates/janus-engine/src/compute/ops/tests.rs:403,430 (the pick on the GPU) and :149-152 (the matrix product)
    assert run_sample(ops, torch.tensor([[-1.0, 0.5, 4.2, 3.9, 2.0]], device=DEV), 0.0) == [2]
    a = torch.tensor([[1., 2., 3.], [4., 5., 6.]], device=DEV)
    b = torch.tensor([[7., 9., 11.], [8., 10., 12.]], device=DEV)
    y = torch.empty(2, 2, device=DEV)
    ops.gemm_f32(a, b, y)
    assert y.flatten().tolist() == [58., 64., 139., 154.]


@pytest.mark.parametrize("V", [384, 5003, 128256])
@pytest.mark.parametrize("top_k, top_p", [(0, 1.0), (40, 1.0), (0, 0.8), (50, 0.9)])
def test_temperature_sampling_follows_the_plain_distribution(ops, V, top_k, top_p):
    B, T = 24, 0.8
    g = torch.Generator().manual_seed(V + top_k)
    logits = (torch.randn(B, V, generator=g) * 2.5).to(DEV)
    got = run_sample(ops, logits, T, top_k, top_p, seed=5)
    for b in range(B):
        probs = P.sampling_distribution(logits[b].cpu(), T, top_k, top_p).double()
        assert probs[got[b]] > 0, f"row {b}: token {got[b]} is outside the kept set"
        cdf = torch.cumsum(probs, 0)
        u = P.uniform_for(5, b, 0)
        lo = float(cdf[got[b]] - probs[got[b]])
        # the token's interval of the cumulative distribution holds u, up to float32 summation order
        assert lo - 2e-4 <= u < float(cdf[got[b]]) + 2e-4, (b, got[b], lo, u, float(cdf[got[b]]))
    # another step draws another number; the same step the same
    assert run_sample(ops, logits, T, top_k, top_p, seed=5) == got
    again = run_sample(ops, logits, T, top_k, top_p, seed=5, steps=torch.ones(B, dtype=torch.int32, device=DEV))
    assert again != got


@pytest.mark.parametrize("V", [5003, 32000])
def test_sampling_with_every_option_draws_from_the_plain_kept_set_at_every_step(ops, V):
    """Repetition penalty, top-k, temperature and top-p together, 40 steps of 16 rows: every drawn token has a
    probability above zero in the plain distribution over the same context, its interval of the cumulative
    distribution holds the step's number, and the kernel's own counts follow what it drew."""
    B, T, top_k, top_p, pen = 16, 0.9, 60, 0.85, 1.3
    g = torch.Generator().manual_seed(V)
    counts = torch.zeros(B, V, dtype=torch.int32, device=DEV)
    context = [[] for _ in range(B)]
    for step in range(40):
        logits = (torch.randn(B, V, generator=g) * 2.0).to(DEV)
        got = run_sample(ops, logits, T, top_k, top_p, penalty=pen, counts=counts, seed=9,
                         steps=torch.full((B,), step, dtype=torch.int32, device=DEV))
        for b in range(B):
            probs = P.sampling_distribution(logits[b].cpu(), T, top_k, top_p, pen, context[b]).double()
            assert probs[got[b]] > 0, f"step {step} row {b}: token {got[b]} is outside the kept set"
            cdf = torch.cumsum(probs, 0)
            u = P.uniform_for(9, b, step)
            assert float(cdf[got[b]] - probs[got[b]]) - 2e-4 <= u < float(cdf[got[b]]) + 2e-4
            context[b].append(got[b])
    want = torch.zeros(B, V, dtype=torch.int32)
    for b in range(B):
        for t in context[b]:
            want[b, t] += 1
    assert torch.equal(counts.cpu(), want)


def test_repetition_penalty_counts(ops):
    V = 300
    logits = torch.zeros(2, V, device=DEV)
    logits[0, 10], logits[0, 20] = 4.0, 3.0
    logits[1, 10], logits[1, 20] = -0.5, -1.0
    logits[1, :10] = -3.0; logits[1, 11:20] = -3.0; logits[1, 21:] = -3.0
    counts = torch.zeros(2, V, dtype=torch.int32, device=DEV)
    assert run_sample(ops, logits, 0.0, penalty=2.0, counts=counts) == [10, 10]
    assert counts[0, 10] == 1 and counts[1, 10] == 1                  # the kernel counted its own picks
    # once counted: 4/2 < 3 and -0.5*2 = -1.0 ties with index 20 -> lowest index (10) still wins row 1
    assert run_sample(ops, logits, 0.0, penalty=2.0, counts=counts) == [20, 10]
    ctx = [[10, 20], [10, 10]]
    want = [P.sample(logits[i].cpu(), 0.0, 0.0, repetition_penalty=2.0, context=ctx[i]) for i in range(2)]
    assert run_sample(ops, logits, 0.0, penalty=2.0, counts=counts) == want
