"""Each CUDA kernel alone against a plain float64 formulation of the same
operation, at sizes other than the tiny models' (odd widths, head sizes in
steps of 16, group sizes 1..8, vocabularies that are no power of two)."""
import math

import numpy as np
import pytest
import torch

import plain_llama as pl

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dt):
    return 2e-6 if dt is torch.float32 else 1.6e-2


def rel_err(got, want):
    want = want.double().cpu()
    return float((got.double().cpu() - want).abs().max() / want.abs().max().clamp_min(1e-30))


@pytest.fixture(scope="module")
def ops():
    from rllm_b200.kernels import ops
    return ops


@pytest.fixture()
def err():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("V,H", [(1000, 72), (37, 2048 + 8)])
def test_embedding(ops, err, dt, V, H):
    torch.manual_seed(0)
    table = torch.randn(V, H, device=DEV).to(dt)
    ids = torch.randint(0, V, (19,), device=DEV, dtype=torch.int32)
    out = torch.empty(19, H, device=DEV)
    ops.embedding(ids, table, out, err)
    assert torch.equal(out, table.float()[ids.long()]) and int(err.item()) == 0
    ids[3] = V
    ops.embedding(ids, table, out, err)
    assert int(err.item()) == 1 and float(out[3].abs().max()) == 0.0      # refused, not read out of bounds


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("wdt", DTYPES)
@pytest.mark.parametrize("H,eps", [(72, 1e-5), (1000, 1e-6), (5120 + 24, 1e-3)])
def test_rmsnorm(ops, dt, wdt, H, eps):
    torch.manual_seed(1)
    x = torch.randn(7, H, device=DEV) * 3
    w = (1 + 0.1 * torch.randn(H, device=DEV)).to(wdt)
    delta = torch.randn(7, H, device=DEV).to(dt)
    want = pl.rms_norm(x.double().cpu(), w.double().cpu(), eps)
    out = torch.empty(7, H, device=DEV, dtype=dt)
    ops.rmsnorm(x, w, eps, out)
    assert rel_err(out, want) <= tol(dt)
    # fused residual add: x += delta (float32), then the norm of the sum
    x2 = x.clone()
    ops.rmsnorm(x2, w, eps, out, delta=delta, writeback=True)
    assert torch.equal(x2, x + delta.float())
    assert rel_err(out, pl.rms_norm((x + delta.float()).double().cpu(), w.double().cpu(), eps)) <= tol(dt)
    # gathered rows, no write-back
    rows = torch.tensor([5, 0, 5], device=DEV, dtype=torch.int32)
    x3 = x.clone()
    out3 = torch.empty(3, H, device=DEV, dtype=dt)
    ops.rmsnorm(x3, w, eps, out3, delta=delta, rows=rows)
    assert torch.equal(x3, x) and torch.equal(out3, out[rows.long()])


@pytest.mark.parametrize("dt", DTYPES)
def test_residual_add_and_silu_mul(ops, dt):
    torch.manual_seed(2)
    x = torch.randn(5, 136, device=DEV)
    d = torch.randn(5, 136, device=DEV).to(dt)
    want = x + d.float()
    ops.residual_add(x, d)
    assert torch.equal(x, want)
    gu = (torch.randn(9, 2 * 200, device=DEV) * 4).to(dt)
    out = torch.empty(9, 200, device=DEV, dtype=dt)
    ops.silu_mul(gu, out)
    g, u = gu.double().cpu()[:, :200], gu.double().cpu()[:, 200:]
    assert rel_err(out, pl.silu(g) * u) <= tol(dt)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,rd,page", [(6, 2, 48, 48, 4), (5, 5, 16, 8, 16), (8, 1, 128, 128, 32), (2, 1, 256, 64, 8)])
def test_rope_and_cache_write(ops, err, dt, nq, nkv, d, rd, page):
    torch.manual_seed(3)
    T, S, pages = 11, 2, 40
    theta = 123456.0
    inv = torch.tensor([theta ** (-(2 * i) / rd) for i in range(rd // 2)], dtype=torch.float64)
    qkv = torch.randn(T, (nq + 2 * nkv) * d, device=DEV).to(dt)
    src = qkv.clone()
    positions = torch.tensor([70000, 70001, 70002, 70003, 70004, 3, 4, 5, 6, 7, 8], dtype=torch.int32, device=DEV)
    token_seq = torch.tensor([0] * 5 + [1] * 6, dtype=torch.int32, device=DEV)
    maxb = 70005 // page + 1
    table = torch.full((S, maxb), -1, dtype=torch.int32, device=DEV)
    perm = torch.randperm(pages)
    table[0, 70000 // page: 70004 // page + 1] = perm[:70004 // page - 70000 // page + 1].int().to(DEV)
    table[1, : 8 // page + 1] = perm[20:20 + 8 // page + 1].int().to(DEV)
    kc = torch.zeros(pages, nkv, page, d, device=DEV, dtype=dt)
    vc = torch.zeros_like(kc)
    ops.rope_kv_write(qkv, positions, token_seq, inv.to(DEV), rd, table, kc, vc, nq, nkv, d, err)
    assert int(err.item()) == 0
    x = src.double().cpu().view(T, nq + 2 * nkv, d)
    def rot(h):
        out = h.clone()
        out[..., :rd] = pl.apply_rope(h[..., :rd], positions.cpu(), inv)
        return out
    assert rel_err(qkv.view(T, nq + 2 * nkv, d)[:, :nq], rot(x[:, :nq])) <= tol(dt)
    k_want, v_want = rot(x[:, nq:nq + nkv]), x[:, nq + nkv:]
    for t in range(T):
        p, s = int(positions[t]), int(token_seq[t])
        pg = int(table[s, p // page])
        assert rel_err(kc[pg, :, p % page], k_want[t]) <= tol(dt)
        assert torch.equal(vc[pg, :, p % page].double().cpu(), v_want[t])
    assert int((kc.abs().sum(dim=(1, 3)) > 0).sum()) == T           # nothing else was written
    # v untouched in the buffer; a token whose page is missing is refused
    assert torch.equal(qkv.view(T, nq + 2 * nkv, d)[:, nq + nkv:], src.view(T, nq + 2 * nkv, d)[:, nq + nkv:])
    table[1, 0] = -1
    ops.rope_kv_write(src.clone(), positions, token_seq, inv.to(DEV), rd, table, kc, vc, nq, nkv, d, err)
    assert int(err.item()) == 2


def paged_case(dt, nq, nkv, d, page, lens, q_lens, pages=64, seed=4, order="random"):
    """Sequences with contexts ``lens`` whose last ``q_lens`` tokens are queries.  ``order``: the pages of a
    sequence in random order, "sequential" (one after the other in the cache, as from a fresh pool) or "runs"
    (one after the other with a stray page now and then)."""
    g = torch.Generator().manual_seed(seed)
    S = len(lens)
    ks = [torch.randn(n, nkv, d, generator=g).to(dt) for n in lens]
    vs = [torch.randn(n, nkv, d, generator=g).to(dt) for n in lens]
    qs = [torch.randn(m, nq, d, generator=g).to(dt) for m in q_lens]
    maxb = max(-(-n // page) for n in lens)
    table = torch.full((S, maxb), -1, dtype=torch.int32)
    perm = torch.randperm(pages, generator=g).tolist() if order == "random" else list(range(pages - 1, -1, -1))
    kc = torch.zeros(pages, nkv, page, d, dtype=dt)
    vc = torch.zeros_like(kc)
    for s, n in enumerate(lens):
        for b in range(-(-n // page)):
            stray = order == "runs" and int(torch.randint(0, 7, (1,), generator=g)) == 0
            pg = perm.pop(int(torch.randint(0, len(perm), (1,), generator=g))) if stray else perm.pop()
            table[s, b] = pg
            m = min(page, n - b * page)
            kc[pg, :, :m] = ks[s][b * page:b * page + m].transpose(0, 1)
            vc[pg, :, :m] = vs[s][b * page:b * page + m].transpose(0, 1)
    positions = torch.cat([torch.arange(n - m, n) for n, m in zip(lens, q_lens)]).int()
    token_seq = torch.cat([torch.full((m,), s) for s, m in enumerate(q_lens)]).int()
    return ks, vs, qs, table, kc, vc, positions, token_seq


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,page,window", [(6, 2, 48, 4, 0), (5, 5, 16, 16, 0), (8, 1, 128, 32, 0),
                                                  (4, 2, 64, 8, 37), (3, 1, 256, 16, 5)])
def test_attention_simt(ops, err, dt, nq, nkv, d, page, window):
    lens, q_lens = [150, 1, 33, 64], [1, 1, 33, 7]
    ks, vs, qs, table, kc, vc, positions, token_seq = paged_case(dt, nq, nkv, d, page, lens, q_lens)
    q = torch.cat(qs).reshape(-1, nq * d).to(DEV)
    out = torch.empty_like(q)
    scale = 0.77 / math.sqrt(d)
    ops.attention_simt(q, nq * d, out, kc.to(DEV), vc.to(DEV), table.to(DEV), positions.to(DEV),
                       token_seq.to(DEV), nq, nkv, d, window, scale, err)
    assert int(err.item()) == 0
    off = 0
    for s, (n, m) in enumerate(zip(lens, q_lens)):
        want = pl.attention(qs[s].double(), ks[s].double(), vs[s].double(), torch.arange(n - m, n),
                            window=window or None, scale=scale)
        assert rel_err(out[off:off + m], want) <= tol(dt), (s, n, m)
        off += m


@pytest.mark.parametrize("dt", DTYPES)
def test_attention_finds_one_far_key(ops, err, dt):
    """One key among hundreds, at the far end of the context and at a page's
    first row, is made to dominate: the output must be its value."""
    nq, nkv, d, page = 4, 2, 32, 16
    lens, q_lens = [700], [1]
    ks, vs, qs, table, kc, vc, positions, token_seq = paged_case(dt, nq, nkv, d, page, lens, q_lens, seed=9)
    for target in (0, 16, 15, 699, 400):
        kc2 = kc.clone()
        qq = qs[0].clone()
        pg = int(table[0, target // page])
        kc2[pg, :, target % page] = 0
        kc2[pg, :, target % page, 0] = 30.0
        qq[:, :, 0] = 30.0
        q = qq.reshape(1, nq * d).to(DEV)
        out = torch.empty_like(q)
        ops.attention_simt(q, nq * d, out, kc2.to(DEV), vc.to(DEV), table.to(DEV), positions.to(DEV),
                           token_seq.to(DEV), nq, nkv, d, 0, 1.0, err)
        want = vs[0][target].repeat_interleave(nq // nkv, dim=0).reshape(1, nq * d)
        assert rel_err(out, want) <= tol(dt), target


@pytest.mark.parametrize("M,N,K", [(1, 130, 72), (7, 389, 96), (64, 64, 16), (129, 200, 1000), (300, 17, 264)])
def test_gemm_f32(ops, M, N, K):
    torch.manual_seed(5)
    a, w = torch.randn(M, K, device=DEV), torch.randn(N, K, device=DEV)
    out = torch.empty(M, N, device=DEV)
    ops.gemm_f32(a, w, out)
    assert rel_err(out, a.double().cpu() @ w.double().cpu().t()) <= 2e-6
    # a row's result does not depend on what else is in the batch
    out1 = torch.empty(1, N, device=DEV)
    ops.gemm_f32(a[M // 2:M // 2 + 1], w, out1)
    assert torch.equal(out1[0], out[M // 2])


def test_sizes_that_kernels_refuse_raise(ops, err):
    from rllm_b200.kernels.ops import KernelError
    q = torch.zeros(1, 2 * 24, device=DEV)
    kc = torch.zeros(4, 1, 16, 24, device=DEV)
    table = torch.zeros(1, 1, dtype=torch.int32, device=DEV)
    z = torch.zeros(1, dtype=torch.int32, device=DEV)
    with pytest.raises(KernelError, match="no kernel"):
        ops.attention_simt(q, 48, torch.empty_like(q), kc, kc, table, z, z, 2, 1, 24, 0, 1.0, err)
    with pytest.raises(KernelError, match="CUDA tensors only"):
        ops.silu_mul(torch.zeros(2, 8), torch.zeros(2, 4))


# ---------------------------------------------------------------------------
# tensor-core attention (bfloat16): prefill and split-KV decode
# ---------------------------------------------------------------------------
MMA_CASES = [(8, 2, 64, 16, 0), (3, 1, 32, 8, 0), (4, 4, 128, 16, 0), (12, 2, 16, 4, 0), (32, 8, 64, 16, 0),
             (8, 2, 64, 16, 300), (6, 2, 128, 32, 70), (5, 1, 32, 8, 17)]


@pytest.mark.parametrize("nq,nkv,d,page,window", MMA_CASES)
def test_attention_prefill_mma(ops, err, nq, nkv, d, page, window):
    dt = torch.bfloat16
    lens, q_lens = [700, 64, 65, 130, 2], [257, 64, 2, 129, 2]        # portions after earlier context, and whole prompts
    ks, vs, qs, table, kc, vc, positions, token_seq = paged_case(dt, nq, nkv, d, page, lens, q_lens, pages=256)
    q = torch.cat(qs).reshape(-1, nq * d).to(DEV)
    out = torch.zeros_like(q)
    q_start = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32, device=DEV)
    seq_lens = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(d)
    ops.attention_prefill_bf16(q, nq * d, out, kc.to(DEV), vc.to(DEV), table.to(DEV), q_start, seq_lens,
                               0, len(lens), sum(q_lens), nq, nkv, d, window, scale, err)
    assert int(err.item()) == 0
    off = 0
    for s, (n, m) in enumerate(zip(lens, q_lens)):
        want = pl.attention(qs[s].double(), ks[s].double(), vs[s].double(), torch.arange(n - m, n),
                            window=window or None, scale=scale)
        assert rel_err(out[off:off + m], want) <= tol(dt), (s, n, m)
        off += m
    # a subrange of the sequences leaves the other rows alone
    out2 = torch.zeros_like(q)
    ops.attention_prefill_bf16(q, nq * d, out2, kc.to(DEV), vc.to(DEV), table.to(DEV), q_start, seq_lens,
                               2, 4, q_lens[2] + q_lens[3], nq, nkv, d, window, scale, err)
    a, b = sum(q_lens[:2]), sum(q_lens[:4])
    assert torch.equal(out2[a:b], out[a:b]) and float(out2[:a].abs().max()) == 0 and float(out2[b:].abs().max()) == 0


TCGEN05_CASES = [(8, 2, 64, 16, 0), (32, 8, 64, 16, 0), (4, 4, 64, 32, 0), (16, 1, 64, 64, 0), (8, 2, 64, 128, 300),
                 (2, 1, 64, 16, 70), (64, 1, 64, 16, 0), (6, 3, 64, 32, 129), (6, 2, 64, 16, 0), (5, 1, 64, 32, 40),
                 (8, 2, 128, 16, 0), (32, 8, 128, 16, 0), (4, 4, 128, 32, 0), (24, 8, 128, 16, 0), (16, 1, 128, 64, 0),
                 (8, 2, 128, 32, 300), (3, 1, 128, 16, 65)]


@pytest.mark.parametrize("order", ["sequential", "runs"])
@pytest.mark.parametrize("nq,nkv,d,page,window", [(32, 8, 64, 16, 0), (6, 3, 64, 32, 129), (16, 1, 64, 64, 0), (8, 2, 64, 128, 0),
                                                  (24, 8, 128, 16, 0), (8, 2, 128, 32, 300), (16, 1, 128, 64, 0)])
def test_attention_prefill_tcgen05_pages_that_follow_one_another(ops, err, nq, nkv, d, page, window, order):
    """Sequences whose pages follow one another in the cache (what a fresh pool hands out), with or without a
    stray page now and then, up to the last page of the pool."""
    dt = torch.bfloat16
    lens, q_lens = [700, 64, 65, 130, 2, 385, 1000], [257, 64, 2, 129, 2, 384, 1000]
    need = sum(-(-n // page) for n in lens)
    ks, vs, qs, table, kc, vc, positions, token_seq = paged_case(dt, nq, nkv, d, page, lens, q_lens, pages=need, order=order)
    T = sum(q_lens)
    q = torch.cat(qs).reshape(T, nq * d).to(DEV)
    out = torch.zeros(T, nq * d, dtype=dt, device=DEV)
    q_start = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32, device=DEV)
    seq_lens = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scale = 1.1 / math.sqrt(d)
    ops.attention_prefill_tcgen05(q, nq * d, out, kc.to(DEV), vc.to(DEV), table.to(DEV), q_start, seq_lens,
                                  0, len(lens), T, nq, nkv, d, window, scale, err)
    assert int(err.item()) == 0
    off = 0
    for s, (n, m) in enumerate(zip(lens, q_lens)):
        want = pl.attention(qs[s].double(), ks[s].double(), vs[s].double(), torch.arange(n - m, n),
                            window=window or None, scale=scale)
        assert rel_err(out[off:off + m], want) <= tol(dt), (s, n, m)
        off += m


@pytest.mark.parametrize("nq,nkv,d,page,window", TCGEN05_CASES)
def test_attention_prefill_tcgen05(ops, err, nq, nkv, d, page, window):
    """The tcgen05 kernel for prompt portions (head size 64): portions after earlier context and whole
    prompts, from 2 tokens to several 128-key tiles, strided q rows as in the engine.  Pages that no
    sequence holds, and the rows of a last page behind a sequence's end, hold NaN: nothing of them
    may reach a result."""
    dt = torch.bfloat16
    lens, q_lens = [700, 64, 65, 130, 2, 385], [257, 64, 2, 129, 2, 384]
    ks, vs, qs, table, kc, vc, positions, token_seq = paged_case(dt, nq, nkv, d, page, lens, q_lens, pages=256)
    held = torch.zeros(256, dtype=torch.bool)
    held[table[table >= 0].long()] = True
    kc[~held] = float("nan")
    vc[~held] = float("nan")
    for s, n in enumerate(lens):
        if n % page:
            kc[int(table[s, n // page]), :, n % page:] = float("nan")
            vc[int(table[s, n // page]), :, n % page:] = float("inf")
    T = sum(q_lens)
    stride = (nq + 2 * nkv) * d
    qkv = torch.randn(T, stride).to(dt).to(DEV)
    qkv[:, : nq * d] = torch.cat(qs).reshape(T, nq * d).to(DEV)
    out = torch.zeros(T, nq * d, dtype=dt, device=DEV)
    q_start = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32, device=DEV)
    seq_lens = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scale = 0.9 / math.sqrt(d)
    assert ops.attention_prefill_tcgen05_supported(nq, nkv, d, page)
    ops.attention_prefill_tcgen05(qkv, stride, out, kc.to(DEV), vc.to(DEV), table.to(DEV), q_start, seq_lens,
                                  0, len(lens), T, nq, nkv, d, window, scale, err)
    assert int(err.item()) == 0
    off = 0
    for s, (n, m) in enumerate(zip(lens, q_lens)):
        want = pl.attention(qs[s].double(), ks[s].double(), vs[s].double(), torch.arange(n - m, n),
                            window=window or None, scale=scale)
        assert rel_err(out[off:off + m], want) <= tol(dt), (s, n, m)
        off += m
    # a subrange of the sequences leaves the other rows alone, and a sequence's rows do not depend on the batch
    out2 = torch.zeros_like(out)
    ops.attention_prefill_tcgen05(qkv, stride, out2, kc.to(DEV), vc.to(DEV), table.to(DEV), q_start, seq_lens,
                                  2, 4, q_lens[2] + q_lens[3], nq, nkv, d, window, scale, err)
    a, b = sum(q_lens[:2]), sum(q_lens[:4])
    assert torch.equal(out2[a:b], out[a:b]) and float(out2[:a].abs().max()) == 0 and float(out2[b:].abs().max()) == 0
    # a portion cut in two gives the same rows: the second half alone, after the first as context
    s, cut = 0, 100
    a = 0
    q_start2 = torch.tensor([0, q_lens[s] - cut], dtype=torch.int32, device=DEV)
    out3 = torch.zeros(q_lens[s] - cut, nq * d, dtype=dt, device=DEV)
    ops.attention_prefill_tcgen05(qkv[a + cut:a + q_lens[s]], stride, out3, kc.to(DEV), vc.to(DEV),
                                  table[s:s + 1].contiguous().to(DEV), q_start2, seq_lens[s:s + 1], 0, 1,
                                  q_lens[s] - cut, nq, nkv, d, window, scale, err)
    assert int(err.item()) == 0
    assert rel_err(out3, out[a + cut:a + q_lens[s]].double().cpu()) <= 2e-3    # other tiles of rows: rounding only


@pytest.mark.parametrize("kind,nq,nkv,d,page,window", [("tcgen05", 4, 2, 64, 16, 0), ("tcgen05", 4, 1, 128, 16, 0),
                                                       ("tcgen05", 4, 2, 64, 16, 900), ("mma", 4, 2, 64, 16, 0),
                                                       ("mma", 6, 2, 32, 8, 0)])
def test_attention_prefill_long_portion(ops, err, kind, nq, nkv, d, page, window):
    """A portion of 1,200 tokens behind 1,800 tokens of context: tens of key tiles a row, the rings of the
    tcgen05 kernel wrapping many times, rows whose max grows late (one far key made to dominate)."""
    dt = torch.bfloat16
    n, m = 3000, 1200
    ks, vs, qs, table, kc, vc, positions, token_seq = paged_case(dt, nq, nkv, d, page, [n], [m],
                                                                 pages=-(-n // page) + 5, seed=12)
    # key 2500 answers the queries from 2600 on with a large score: their running max jumps late
    qs[0][800:, :, 5] = 12.0
    pg = int(table[0, 2500 // page])
    ks[0][2500] = 0
    ks[0][2500, :, 5] = 12.0
    kc[pg, :, 2500 % page] = ks[0][2500]
    q = qs[0].reshape(m, nq * d).to(DEV)
    out = torch.zeros_like(q)
    q_start = torch.tensor([0, m], dtype=torch.int32, device=DEV)
    seq_lens = torch.tensor([n], dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(d)
    fn = ops.attention_prefill_tcgen05 if kind == "tcgen05" else ops.attention_prefill_bf16
    fn(q, nq * d, out, kc.to(DEV), vc.to(DEV), table.to(DEV), q_start, seq_lens, 0, 1, m, nq, nkv, d, window, scale, err)
    assert int(err.item()) == 0
    want = pl.attention(qs[0].double(), ks[0].double(), vs[0].double(), torch.arange(n - m, n),
                        window=window or None, scale=scale)
    for a in range(0, m, 300):
        assert rel_err(out[a:a + 300], want[a:a + 300]) <= tol(dt), a


def test_tcgen05_attention_refuses_other_sizes(ops, err):
    from rllm_b200.kernels.ops import KernelError
    assert not ops.attention_prefill_tcgen05_supported(8, 2, 32, 16)      # head size
    assert not ops.attention_prefill_tcgen05_supported(8, 2, 128, 128)    # a page larger than a key tile
    assert not ops.attention_prefill_tcgen05_supported(8, 2, 64, 8)
    q = torch.zeros(4, 8 * 128, device=DEV, dtype=torch.bfloat16)
    kc = torch.zeros(4, 2, 128, 128, device=DEV, dtype=torch.bfloat16)
    table = torch.zeros(1, 1, dtype=torch.int32, device=DEV)
    qs = torch.tensor([0, 4], dtype=torch.int32, device=DEV)
    sl = torch.tensor([4], dtype=torch.int32, device=DEV)
    with pytest.raises(KernelError, match="no kernel"):
        ops.attention_prefill_tcgen05(q, 8 * 128, torch.empty_like(q), kc, kc, table, qs, sl, 0, 1, 4, 8, 2, 128, 0, 1.0, err)


@pytest.mark.parametrize("nq,nkv,d,page,window", MMA_CASES)
def test_attention_decode_mma(ops, err, nq, nkv, d, page, window):
    dt = torch.bfloat16
    lens = [1, 255, 256, 257, 1000, 64, 513]
    q_lens = [1] * len(lens)
    ks, vs, qs, table, kc, vc, positions, token_seq = paged_case(dt, nq, nkv, d, page, lens, q_lens, pages=1024)
    q = torch.cat(qs).reshape(-1, nq * d).to(DEV)
    seq_lens = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(d)
    outs = []
    for bound in (max(lens), 4096):          # the bound on the lengths (as under a CUDA graph) changes nothing
        out = torch.zeros_like(q)
        ops.attention_decode_bf16(q, nq * d, out, kc.to(DEV), vc.to(DEV), table.to(DEV), seq_lens, len(lens), bound,
                                  nq, nkv, d, window, scale, err)
        outs.append(out)
    assert int(err.item()) == 0 and torch.equal(outs[0], outs[1])
    for s, n in enumerate(lens):
        want = pl.attention(qs[s].double(), ks[s].double(), vs[s].double(), torch.tensor([n - 1]),
                            window=window or None, scale=scale)
        assert rel_err(outs[0][s:s + 1], want) <= tol(dt), (s, n)
    # a sequence's row does not depend on the batch it is in
    alone = torch.zeros(1, nq * d, device=DEV, dtype=dt)
    ops.attention_decode_bf16(q[4:5], nq * d, alone, kc.to(DEV), vc.to(DEV), table[4:5].contiguous().to(DEV),
                              seq_lens[4:5], 1, 1000, nq, nkv, d, window, scale, err)
    assert torch.equal(alone[0], outs[0][4])


@pytest.mark.parametrize("nq,nkv,d,page,window", [(8, 2, 64, 16, 0), (8, 2, 64, 16, 5000), (4, 1, 128, 32, 0), (6, 3, 32, 8, 0),
                                                  (8, 2, 128, 16, 0), (6, 2, 128, 64, 3000)])
def test_attention_decode_long_sequences(ops, err, nq, nkv, d, page, window):
    """Tens of CTAs a (sequence, kv head): their results are merged in several rounds of eight and two
    halves; beside them short sequences whose CTAs mostly have nothing to do."""
    dt = torch.bfloat16
    lens = [9300, 17, 4097, 20000, 512]
    ks, vs, qs, table, kc, vc, positions, token_seq = paged_case(dt, nq, nkv, d, page, lens, [1] * len(lens),
                                                                 pages=sum(-(-n // page) for n in lens) + 3, seed=6)
    q = torch.cat(qs).reshape(-1, nq * d).to(DEV)
    seq_lens = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(d)
    out = torch.zeros_like(q)
    ops.attention_decode_bf16(q, nq * d, out, kc.to(DEV), vc.to(DEV), table.to(DEV), seq_lens, len(lens), 20480,
                              nq, nkv, d, window, scale, err)
    assert int(err.item()) == 0
    for s, n in enumerate(lens):
        want = pl.attention(qs[s].double(), ks[s].double(), vs[s].double(), torch.tensor([n - 1]),
                            window=window or None, scale=scale)
        assert rel_err(out[s:s + 1], want) <= tol(dt), (s, n)
    # one key far back made to dominate, in a late round of the merge
    if window == 0:
        target = 13000
        kc2, qq = kc.clone(), qs[3].clone()
        pg = int(table[3, target // page])
        kc2[pg, :, target % page] = 0
        kc2[pg, :, target % page, 3] = 30.0
        qq[:, :, 3] = 30.0
        q2 = q.clone()
        q2[3] = qq.reshape(nq * d).to(DEV)
        out2 = torch.zeros_like(q)
        ops.attention_decode_bf16(q2, nq * d, out2, kc2.to(DEV), vc.to(DEV), table.to(DEV), seq_lens, len(lens), 20480,
                                  nq, nkv, d, 0, 1.0, err)
        want = vs[3][target].repeat_interleave(nq // nkv, dim=0).reshape(1, nq * d)
        assert rel_err(out2[3:4], want) <= tol(dt)


@pytest.mark.parametrize("kind", ["prefill", "decode", "tcgen05", "decode_many_64", "decode_many_128"])
def test_mma_attention_finds_one_far_key(ops, err, kind):
    """One key among a thousand, at a tile's, split's or page's edge, is made to
    dominate: the output must be its value.  The "many" kinds give the decode kernel
    a bound on the length so large that it takes the tiling it uses for large batches
    (tiles of 16 keys for heads of 128)."""
    dt = torch.bfloat16
    nq, nkv, d, page = (4, 2, 128, 16) if kind == "decode_many_128" else (8, 2, 64, 16)
    n = 1100
    bound = 65536 if kind.startswith("decode_many") else n
    m = {"prefill": 5, "tcgen05": 40}.get(kind, 1)
    ks, vs, qs, table, kc, vc, positions, token_seq = paged_case(dt, nq, nkv, d, page, [n], [m], pages=128, seed=9)
    seq_lens = torch.tensor([n], dtype=torch.int32, device=DEV)
    q_start = torch.tensor([0, m], dtype=torch.int32, device=DEV)
    for target in (0, 15, 16, 31, 32, 47, 48, 63, 64, 127, 128, 143, 144, 255, 256, 511, 512, 1023, 1024, 1039, 1040,
                   n - m - 1, n - m):
        kc2, qq = kc.clone(), qs[0].clone()
        pg = int(table[0, target // page])
        kc2[pg, :, target % page] = 0
        kc2[pg, :, target % page, 3] = 30.0
        qq[:, :, 3] = 30.0
        q = qq.reshape(m, nq * d).to(DEV)
        out = torch.zeros_like(q)
        if kind.startswith("decode"):
            ops.attention_decode_bf16(q, nq * d, out, kc2.to(DEV), vc.to(DEV), table.to(DEV), seq_lens, 1, bound,
                                      nq, nkv, d, 0, 1.0, err)
        else:
            fn = ops.attention_prefill_tcgen05 if kind == "tcgen05" else ops.attention_prefill_bf16
            fn(q, nq * d, out, kc2.to(DEV), vc.to(DEV), table.to(DEV), q_start, seq_lens,
               0, 1, m, nq, nkv, d, 0, 1.0, err)
        want = vs[0][target].repeat_interleave(nq // nkv, dim=0).reshape(1, nq * d).expand(m, -1)
        assert rel_err(out, want) <= tol(dt), target


@pytest.mark.parametrize("kind,d,dt", [("simt", 48, torch.float32), ("simt", 64, torch.bfloat16), ("prefill", 64, torch.bfloat16),
                                       ("tcgen05", 64, torch.bfloat16), ("tcgen05", 128, torch.bfloat16),
                                       ("decode", 64, torch.bfloat16), ("decode", 128, torch.bfloat16)])
def test_a_dominant_key_at_the_windows_edge(ops, err, kind, d, dt):
    """A window of 129 keys over a context of 700: the key that is made to dominate lies just outside or just
    inside the window of the first and of the last query row, and at the tile and page edges between; a row
    that sees it returns its value, a row that does not must show no trace of it.  The pages that lie
    wholly ahead of every row's window are given back (-1 in the block table) and hold NaN."""
    nq, nkv, page, window, n = (4, 2, 16, 129, 700) if d == 128 else (6, 2, 16, 129, 700)
    m = 1 if kind == "decode" else 40
    ks, vs, qs, table, kc, vc, positions, token_seq = paged_case(dt, nq, nkv, d, page, [n], [m], pages=64, seed=17)
    first_seen = (n - m) - window + 1                       # the first key that the first row sees
    for b in range(first_seen // page):                     # pages wholly ahead of it
        pg = int(table[0, b])
        kc[pg] = float("nan")
        vc[pg] = float("nan")
        table[0, b] = -1
    seq_lens = torch.tensor([n], dtype=torch.int32, device=DEV)
    q_start = torch.tensor([0, m], dtype=torch.int32, device=DEV)
    kc_d, vc_d, table_d = kc.to(DEV), vc.to(DEV), table.to(DEV)
    qq = qs[0].clone()
    qq[:, :, 3] = 30.0
    q = qq.reshape(m, nq * d).to(DEV)
    pos = torch.arange(n - m, n)
    targets = sorted({t for p in (n - m, n - 1) for t in (p - window, p - window + 1, p - window + 2, p)}
                     | {first_seen + 16 - first_seen % 16, 639, 640, n - m - 1, n - 20})
    for target in targets:
        if target < first_seen - first_seen % page:         # its page has been given back
            continue
        kc2, k2 = kc_d.clone(), ks[0].clone()
        pg = int(table[0, target // page])
        assert pg >= 0
        kc2[pg, :, target % page] = 0
        kc2[pg, :, target % page, 3] = 30.0
        k2[target] = 0
        k2[target, :, 3] = 30.0
        out = torch.zeros_like(q)
        if kind == "decode":
            ops.attention_decode_bf16(q, nq * d, out, kc2, vc_d, table_d, seq_lens, 1, n, nq, nkv, d, window, 1.0, err)
        elif kind == "simt":
            ops.attention_simt(q, nq * d, out, kc2, vc_d, table_d, positions.to(DEV), token_seq.to(DEV),
                               nq, nkv, d, window, 1.0, err)
        else:
            fn = ops.attention_prefill_tcgen05 if kind == "tcgen05" else ops.attention_prefill_bf16
            fn(q, nq * d, out, kc2, vc_d, table_d, q_start, seq_lens, 0, 1, m, nq, nkv, d, window, 1.0, err)
        k_ref, v_ref = k2.double(), vs[0].double()
        k_ref[:first_seen - first_seen % page] = 0           # never seen by any row: any finite value will do
        v_ref[:first_seen - first_seen % page] = 0
        want = pl.attention(qq.double(), k_ref, v_ref, pos, window=window, scale=1.0)
        sees = (pos - window + 1 <= target) & (target <= pos)
        # float32: a score s is rounded to 2^-24 |s| before its exponential is taken, and the scores here are
        # large by construction (the rows that do not see the key still multiply by q's 30)
        smax = float(torch.einsum("mhd,nhd->mhn", qq.double(), k_ref.repeat_interleave(nq // nkv, dim=1)).abs().max())
        bound = max(tol(dt), 4 * smax * 2.0 ** -23)
        assert rel_err(out, want) <= bound, (target, int(sees.sum()), smax)
        if sees.any():                                        # and the rows that see it return its value
            val = vs[0][target].repeat_interleave(nq // nkv, dim=0).reshape(1, nq * d).double()
            assert rel_err(out[sees.to(out.device)], val.expand(int(sees.sum()), -1)) <= tol(dt), target
    assert int(err.item()) == 0


@pytest.mark.parametrize("kind,d", [("decode", 64), ("decode", 128), ("tcgen05", 64), ("tcgen05", 128), ("prefill", 64)])
def test_attention_finds_one_key_among_forty_thousand(ops, err, kind, d):
    """A context of 40,003 keys in 2,501 pages scattered over the cache (313 tiles of 128 keys, 1,251 chunks of
    a decode warp): one key at a time is made to dominate, at the very start, around 2^15, at tile and page
    edges in the middle and at the end; the output must be its value for every query row."""
    dt = torch.bfloat16
    nq, nkv, page = (4, 2, 16) if d == 128 else (8, 2, 16)
    n = 40_003
    m = 1 if kind == "decode" else 37
    ks, vs, qs, table, kc, vc, positions, token_seq = paged_case(dt, nq, nkv, d, page, [n], [m], pages=2600, seed=12)
    seq_lens = torch.tensor([n], dtype=torch.int32, device=DEV)
    q_start = torch.tensor([0, m], dtype=torch.int32, device=DEV)
    kc_d, vc_d, table_d = kc.to(DEV), vc.to(DEV), table.to(DEV)
    qq = qs[0].clone()
    qq[:, :, 3] = 30.0
    q = qq.reshape(m, nq * d).to(DEV)
    for target in (0, 1, 127, 128, 4095, 4096, 20_000, 32_767, 32_768, 32_769, 39_935, 39_936, n - m - 1, n - m):
        kc2 = kc_d.clone()
        pg = int(table[0, target // page])
        kc2[pg, :, target % page] = 0
        kc2[pg, :, target % page, 3] = 30.0
        out = torch.zeros_like(q)
        if kind == "decode":
            ops.attention_decode_bf16(q, nq * d, out, kc2, vc_d, table_d, seq_lens, 1, n, nq, nkv, d, 0, 1.0, err)
        else:
            fn = ops.attention_prefill_tcgen05 if kind == "tcgen05" else ops.attention_prefill_bf16
            fn(q, nq * d, out, kc2, vc_d, table_d, q_start, seq_lens, 0, 1, m, nq, nkv, d, 0, 1.0, err)
        want = vs[0][target].repeat_interleave(nq // nkv, dim=0).reshape(1, nq * d).expand(m, -1)
        assert rel_err(out, want) <= tol(dt), target
    assert int(err.item()) == 0


@pytest.mark.parametrize("nq,nkv,d,rd,page,window", [(8, 2, 64, 64, 16, 0), (3, 1, 32, 16, 8, 0), (4, 4, 128, 128, 16, 40),
                                                     (12, 2, 16, 16, 4, 0), (24, 8, 128, 128, 16, 0), (6, 2, 128, 64, 32, 0)])
def test_decode_with_fused_rotation_and_cache_write(ops, err, nq, nkv, d, rd, page, window):
    """The decode kernel that also rotates the token's q and k and stores k and v
    gives what the separate rotation-and-write kernel followed by attention gives."""
    dt = torch.bfloat16
    lens = [1, 32, 33, 256, 257, 700, 1025]
    S = len(lens)
    ks, vs, qs, table, kc, vc, positions, token_seq = paged_case(dt, nq, nkv, d, page, lens, [1] * S, pages=1024)
    torch.manual_seed(7)
    qkv = torch.randn(S, (nq + 2 * nkv) * d, device=DEV).to(dt)
    inv = torch.tensor([50000.0 ** (-(2 * i) / rd) for i in range(rd // 2)], dtype=torch.float64, device=DEV)
    seq_lens = torch.tensor(lens, dtype=torch.int32, device=DEV)
    pos, tseq, tab = positions.to(DEV), token_seq.to(DEV), table.to(DEV)
    scale = 1.0 / math.sqrt(d)
    # separate kernels
    qa, ka, va = qkv.clone(), kc.to(DEV), vc.to(DEV)
    ops.rope_kv_write(qa, pos, tseq, inv, rd, tab, ka, va, nq, nkv, d, err)
    out_a = torch.zeros(S, nq * d, device=DEV, dtype=dt)
    ops.attention_decode_bf16(qa, qa.shape[1], out_a, ka, va, tab, seq_lens, S, max(lens), nq, nkv, d, window, scale, err)
    # one kernel
    qb, kb, vb = qkv.clone(), kc.to(DEV), vc.to(DEV)
    out_b = torch.zeros_like(out_a)
    ops.attention_decode_bf16(qb, qb.shape[1], out_b, kb, vb, tab, seq_lens, S, max(lens), nq, nkv, d, window, scale, err,
                              inv_freq=inv, rotary_dim=rd, write_kv=True)
    assert int(err.item()) == 0
    assert torch.equal(ka, kb) and torch.equal(va, vb)
    assert torch.equal(out_a, out_b)
    assert torch.equal(qb, qkv)                         # the fused kernel leaves its input alone
    # and against the plain formulation, with the new key and value in place
    x = qkv.double().cpu().view(S, nq + 2 * nkv, d)
    for s, n in enumerate(lens):
        def rot(h):
            o = h.clone()
            o[..., :rd] = pl.apply_rope(h[..., :rd], torch.tensor([n - 1]), inv.cpu())
            return o
        k_all = torch.cat([ks[s][:n - 1].double(), rot(x[s:s + 1, nq:nq + nkv])])
        v_all = torch.cat([vs[s][:n - 1].double(), x[s:s + 1, nq + nkv:]])
        want = pl.attention(rot(x[s:s + 1, :nq]), k_all, v_all, torch.tensor([n - 1]), window=window or None, scale=scale)
        assert rel_err(out_b[s:s + 1], want) <= tol(dt), (s, n)


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(389, 96), (3072, 2048), (17, 264), (256, 64), (2048, 8192)])
def test_gemm_small_m(ops, M, N, K):
    torch.manual_seed(M * 1000 + N)
    x = torch.randn(M, K, device=DEV).bfloat16()
    w = (torch.randn(N, K, device=DEV) * 0.05).bfloat16()
    want = x.double().cpu() @ w.double().cpu().t()
    for dt in (torch.float32, torch.bfloat16):
        out = torch.full((M, N), float("nan"), device=DEV, dtype=dt)
        ops.gemm_small_m(x, w, out)
        assert rel_err(out, want) <= (1e-5 if dt is torch.float32 else 1e-2)
    # a row's result does not depend on the rows around it
    out = torch.empty(M, N, device=DEV)
    ops.gemm_small_m(x, w, out)
    one = torch.empty(1, N, device=DEV)
    ops.gemm_small_m(x[M // 2:M // 2 + 1], w, one)
    assert torch.equal(one[0], out[M // 2])
    # rows of a wider buffer (a view with a row stride)
    wide = torch.randn(M, K + 24, device=DEV).bfloat16()
    ops.gemm_small_m(wide[:, 8:8 + K], w, out)
    assert rel_err(out, wide[:, 8:8 + K].double().cpu() @ w.double().cpu().t()) <= 1e-5


@pytest.mark.parametrize("M", [1, 8, 11, 16])
@pytest.mark.parametrize("I,K", [(176, 64), (264, 96), (8192, 2048), (50, 72)])
def test_gemm_small_m_silu(ops, M, I, K):
    torch.manual_seed(I + M)
    x = torch.randn(M, K, device=DEV).bfloat16()
    w = (torch.randn(2 * I, K, device=DEV) * 0.1).bfloat16()
    out = torch.full((M, I), float("nan"), device=DEV, dtype=torch.bfloat16)
    ops.gemm_small_m(x, w, out, "silu_mul")
    xd, wd = x.double().cpu(), w.double().cpu()
    want = pl.silu(xd @ wd[:I].t()) * (xd @ wd[I:].t())
    assert rel_err(out, want) <= 1e-2


@pytest.mark.parametrize("wdt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,H,K,N2", [(1, 136, 264, 200), (3, 2048, 8192, 3072), (8, 72, 40, 50), (5, 96, 264, 389),
                                       (9, 136, 264, 200), (13, 2048, 8192, 3072), (16, 72, 40, 50),
                                       (8, 2048, 264, 16384), (2, 1024, 72, 13000)])   # grids that run as one wave of the lighter form
def test_gemm_small_m_residual_then_rstd(ops, M, H, K, N2, wdt):
    """The pair of products that stands for 'add into the residual stream, RMSNorm, next product':
    h += x W1^T with the rows' partial sums of squares and h * w_norm on the side, then
    (h w_norm) W2^T scaled by the rows' 1 / rms, compared with the plain formulas."""
    torch.manual_seed(M + H)
    eps = 3e-4
    x = torch.randn(M, K, device=DEV).bfloat16()
    w1 = (torch.randn(H, K, device=DEV) * 0.1).bfloat16()
    h0 = torch.randn(M, H, device=DEV) * 3
    wn = (1 + 0.1 * torch.randn(H, device=DEV)).to(wdt)
    h = h0.clone()
    parts, scaled = ops.gemm_small_m_residual(x, w1, h, wn)
    want_h = h0.double().cpu() + x.double().cpu() @ w1.double().cpu().t()
    assert rel_err(h, want_h) <= 2e-6
    assert rel_err(parts.sum(dim=0), (h.double().cpu() ** 2).sum(dim=1)) <= 1e-6
    assert torch.equal(scaled, (h * wn.float()).bfloat16())
    # without a norm named: no scaled copy, the same h
    h2 = h0.clone()
    parts2, none = ops.gemm_small_m_residual(x, w1, h2, None)
    assert none is None and torch.equal(h2, h) and torch.equal(parts2, parts)
    # the product after the norm: plain, and with the SiLU gate
    want_x = pl.rms_norm(h.double().cpu(), wn.double().cpu(), eps)
    w2 = (torch.randn(N2, H, device=DEV) * 0.1).bfloat16()
    out = torch.full((M, N2), float("nan"), device=DEV, dtype=torch.bfloat16)
    ops.gemm_small_m_rstd(scaled, parts, eps, w2, out)
    assert rel_err(out, want_x @ w2.double().cpu().t()) <= 1e-2
    I = N2 // 2
    act = torch.full((M, I), float("nan"), device=DEV, dtype=torch.bfloat16)
    ops.gemm_small_m_rstd(scaled, parts, eps, w2[:2 * I], act, "silu_mul")
    w2d = w2.double().cpu()
    assert rel_err(act, pl.silu(want_x @ w2d[:I].t()) * (want_x @ w2d[I:2 * I].t())) <= 1e-2
    # a row's results do not depend on the rows beside it
    if M > 1:
        h1 = h0[M - 1:].clone()
        p1, s1 = ops.gemm_small_m_residual(x[M - 1:], w1, h1, wn)
        assert torch.equal(h1[0], h[M - 1]) and torch.equal(p1[:, 0], parts[:, M - 1]) and torch.equal(s1[0], scaled[M - 1])
        o1 = torch.empty(1, N2, device=DEV, dtype=torch.bfloat16)
        ops.gemm_small_m_rstd(s1, p1, eps, w2, o1)
        assert torch.equal(o1[0], out[M - 1])


@pytest.mark.parametrize("M,N,K", [(17, 96, 64), (128, 128, 64), (129, 389, 96), (200, 300, 264), (300, 3072, 2048),
                                   (2048, 2048, 8192), (64, 128256, 2048), (1000, 72, 1000)])
def test_gemm_tcgen05(ops, M, N, K):
    torch.manual_seed(M + N)
    x = torch.randn(M, K, device=DEV).bfloat16()
    w = (torch.randn(N, K, device=DEV) * 0.05).bfloat16()
    want = x.double().cpu() @ w.double().cpu().t() if M * N * K < 2e10 else (x.float() @ w.float().t()).double().cpu()
    for dt in (torch.float32, torch.bfloat16):
        out = torch.full((M, N), float("nan"), device=DEV, dtype=dt)
        ops.gemm_tcgen05(x, w, out)
        ops.check_gemm_errors(torch.device(DEV))
        assert rel_err(out, want) <= (2e-5 if dt is torch.float32 else 1e-2)
    # rows of a wider buffer (a view with a row stride), as the attention output is read
    wide = torch.randn(M, K + 24, device=DEV).bfloat16()
    out = torch.empty(M, N, device=DEV)
    ops.gemm_tcgen05(wide[:, 8:8 + K], w, out)
    assert rel_err(out, (wide[:, 8:8 + K].float() @ w.float().t())) <= 2e-5


@pytest.mark.parametrize("M,I,K", [(33, 176, 64), (130, 264, 96), (2048, 8192, 2048), (257, 50, 72)])
def test_gemm_tcgen05_silu(ops, M, I, K):
    torch.manual_seed(I + M)
    x = torch.randn(M, K, device=DEV).bfloat16()
    w = (torch.randn(2 * I, K, device=DEV) * 0.1).bfloat16()
    out = torch.full((M, I), float("nan"), device=DEV, dtype=torch.bfloat16)
    ops.gemm_tcgen05(x, w, out, "silu_mul")
    ops.check_gemm_errors(torch.device(DEV))
    xf, wf = x.float(), w.float()
    want = pl.silu((xf @ wf[:I].t()).double().cpu()) * (xf @ wf[I:].t()).double().cpu()
    assert rel_err(out, want) <= 1e-2


@pytest.mark.parametrize("n", [1, 3, 4, 1021, 4096, 300_001])
def test_random_weights_are_the_same_bits_on_the_gpu_and_on_the_cpu(ops, n):
    """The kernel of the random-weights mode against its NumPy twin: float32 and bfloat16, both rules,
    lengths that are no multiple of four; and whole tensors through ``draw_tensor``."""
    from rllm_b200.weights import counter_rng as cr
    key = 0x9E3779B97F4A7C15 ^ n
    for one_plus, std in ((False, 0.02), (True, 0.1)):
        want = torch.from_numpy(cr.normal(n, key, std, one_plus))
        got = torch.empty(n, dtype=torch.float32, device=DEV)
        ops.draw_normal(got, key, std, one_plus)
        assert torch.equal(got.cpu(), want), (n, one_plus, (got.cpu() != want).sum())
        got16 = torch.empty(n, dtype=torch.bfloat16, device=DEV)
        ops.draw_normal(got16, key, std, one_plus)
        assert torch.equal(got16.cpu(), want.to(torch.bfloat16))
    ints = torch.empty(n, dtype=torch.int32, device=DEV)
    ops.draw_randint(ints, key, 389)
    assert torch.equal(ints.cpu(), torch.from_numpy(cr.randint(n, key, 389)))


def test_draw_tensor_on_the_device_is_the_written_folder():
    from rllm_b200.parts.spec import TensorSpec
    from rllm_b200.weights import draw_tensor
    for spec in (TensorSpec("model.layers.3.mlp.up_proj.weight", (264, 96)),
                 TensorSpec("model.norm.weight", (96,), role="vector", init=("one_plus_normal", 0.1)),
                 TensorSpec("table", (50,), role="int", init=("randint", 11))):
        assert torch.equal(draw_tensor(spec, 2, str(DEV)).cpu(), draw_tensor(spec, 2))
