"""Each CUDA kernel alone against its plain reference (`plain_ops.PlainOps` on CPU copies), at sizes other than the
engine's: widths and vocabularies that are no power of two, odd head counts and groups, head sizes in steps of 16."""
import math
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from plain_ops import PlainOps

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def ops_pair(dtype):
    from fusezap_core_b200.kernels import cuda_ops
    return cuda_ops(dtype), PlainOps(DT[dtype])


def close(got: torch.Tensor, ref: torch.Tensor, dtype: str, scale: float | None = None, steps: float = 2.0):
    got, ref = got.float().cpu(), ref.float().cpu()
    s = float(ref.abs().max()) if scale is None else scale
    tol = 1e-5 * max(s, 1.0) if dtype == "float32" else steps * 2.0 ** -8 * max(s, 1e-3)
    err = float((got - ref).abs().max())
    assert torch.isfinite(got).all() and err <= tol, f"max |diff| {err:.3e} > {tol:.3e} (scale {s:.3g})"


class Meta:
    """Step metadata for kernel tests: the views the kernels read, on any device."""
    def __init__(self, pos, seq_row, table, device, cut_keys=True, heads=32, items=16):
        from fusezap_core_b200.kernels.table import AttentionPlan, attention_tiles
        self.cut_keys, self.heads, self.items = cut_keys, heads, items
        self.pos = torch.tensor(pos, dtype=torch.int32, device=device)
        self.seq_row = torch.tensor(seq_row, dtype=torch.int32, device=device)
        self._table = torch.tensor(table, dtype=torch.int32, device=device)
        # portions = runs of rows of one request at consecutive positions: (first row, rows, first position, slot)
        segs, i = {}, 0
        while i < len(pos):
            j = i
            while j + 1 < len(pos) and seq_row[j + 1] == seq_row[i] and pos[j + 1] == pos[j] + 1:
                j += 1
            if seq_row[i] >= 0:
                segs[seq_row[i]] = (i, j - i + 1, pos[i], -1)
            i = j + 1
        seg = [segs.get(s, (0, 0, 0, -1)) for s in range(len(table))]
        tiles, cuts, short = attention_tiles([(s, n, p0) for s, (r0, n, p0, _) in enumerate(seg)], len(pos), cut_keys, heads, items)
        self.seg = torch.tensor(seg, dtype=torch.int32, device=device)
        self.plan = AttentionPlan(torch.tensor(tiles or [(-1, 0, -1)], dtype=torch.int32, device=device), len(tiles), short,
                                  torch.tensor(cuts or [(0, 0)], dtype=torch.int32, device=device), len(cuts),
                                  sum(c for _, c in cuts), single_tokens=all(v[1] == 1 for v in segs.values()))
        self.max_context = max(pos) + 1
    def table(self, group):
        return self._table
    def to(self, device):
        return Meta(self.pos.tolist(), self.seq_row.tolist(), self._table.tolist(), device, self.cut_keys, self.heads, self.items)


def make_cache(pages, hkv, bs, hd, dtype, device, write=True):
    pool = torch.zeros(pages, 2, hkv, bs, hd, dtype=dtype, device=device)
    return SimpleNamespace(keys=pool[:, 0], values=pool[:, 1], group=0, page_size=bs, write=write, pool=pool)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embed(dtype):
    cu, pl = ops_pair(dtype)
    g = torch.Generator().manual_seed(0)
    table = torch.randn(509, 72, generator=g).to(DT[dtype])
    tok = torch.randint(0, 509, (37,), generator=g, dtype=torch.int32)
    x, xr = torch.empty(37, 72, device="cuda"), torch.empty(37, 72)
    cu.embed(table.cuda(), tok.cuda(), x)
    pl.embed(table, tok, xr)
    assert torch.equal(x.cpu(), xr)
    cu.check_errors()
    # some rows take their token from another buffer on the device (the ids the step before chose)
    src = torch.full((37,), -1, dtype=torch.int32); src[[0, 9, 36]] = torch.tensor([4, 0, 2], dtype=torch.int32)
    prev = torch.tensor([100, 7, 508, 3, 250], dtype=torch.int32)
    cu.embed(table.cuda(), tok.cuda(), x, src.cuda(), prev.cuda())
    pl.embed(table, tok, xr, src, prev)
    assert torch.equal(x.cpu(), xr) and torch.equal(xr[9], table[100].float()) and torch.equal(xr[1], table[tok[1]].float())
    cu.check_errors()
    bad = tok.clone(); bad[5] = 509
    cu.embed(table.cuda(), bad.cuda(), x)
    from fusezap_core_b200.kernels.table import KernelError
    with pytest.raises(KernelError, match="embedding table"):
        cu.check_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("D", [72, 1000, 4096 + 8])
def test_add_rmsnorm(dtype, D):
    cu, pl = ops_pair(dtype)
    g = torch.Generator().manual_seed(D)
    x, d = torch.randn(19, D, generator=g) * 3, torch.randn(19, D, generator=g)
    for wdt in (torch.float32, DT[dtype]):
        w = (1 + 0.1 * torch.randn(D, generator=g)).to(wdt)
        xc, xp = x.clone().cuda(), x.clone()
        h, hp = torch.empty(19, D, dtype=DT[dtype], device="cuda"), torch.empty(19, D, dtype=DT[dtype])
        cu.add_rmsnorm(xc, d.cuda(), w.cuda(), 1e-5, h)
        pl.add_rmsnorm(xp, d, w, 1e-5, hp)
        assert torch.equal(xc.cpu(), xp), "the residual stream must be x + delta exactly"
        close(h, hp, dtype)
        # no delta; and selected rows with one left out
        cu.add_rmsnorm(xc, None, w.cuda(), 1e-5, h)
        pl.add_rmsnorm(xp, None, w, 1e-5, hp)
        close(h, hp, dtype)
        # weights that do not start on a 16-byte boundary: the kernel that reads them one by one, with the same bits
        w_off = torch.cat([w[:1], w]).cuda()[1:]
        h_off = torch.empty_like(h)
        cu.add_rmsnorm(xc, None, w_off, 1e-5, h_off)
        assert torch.equal(h_off, h), "unaligned weights"
        rows = torch.tensor([18, 0, -1, 7], dtype=torch.int32)
        hr, hrp = torch.empty(4, D, dtype=DT[dtype], device="cuda"), torch.empty(4, D, dtype=DT[dtype])
        before = xc.clone()
        cu.add_rmsnorm(xc, d.cuda(), w.cuda(), 1e-5, hr, rows.cuda())
        pl.add_rmsnorm(xp, d, w, 1e-5, hrp, rows)
        assert torch.equal(xc, before), "row selection must not write x"
        close(hr, hrp, dtype)
        assert float(hr[2].float().abs().max()) == 0.0
    cu.check_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,N,K", [(1, 130, 72), (5, 509, 96), (16, 64, 40), (17, 200, 33), (70, 67, 129), (200, 384, 256)])
def test_linear(dtype, M, N, K):
    cu, pl = ops_pair(dtype)
    g = torch.Generator().manual_seed(M * N + K)
    a, w = torch.randn(M, K, generator=g).to(DT[dtype]), torch.randn(N, K, generator=g).to(DT[dtype])
    b = torch.randn(N, generator=g)
    for out_dt in {torch.float32, DT[dtype]}:
        for bias in (None, b):
            o, op = torch.empty(M, N, dtype=out_dt, device="cuda"), torch.empty(M, N, dtype=out_dt)
            cu.linear(a.cuda(), w.cuda(), None if bias is None else bias.cuda(), o)
            pl.linear(a, w, bias, op)
            close(o, op, "float32" if out_dt == torch.float32 else dtype, scale=math.sqrt(K) * 3)


def test_linear_rows_do_not_depend_on_the_batch():
    """float32: a row's bits are the same alone, among few rows and among many (one fixed order of the k sum)."""
    cu, _ = ops_pair("float32")
    g = torch.Generator().manual_seed(1)
    a, w = torch.randn(150, 200, generator=g).cuda(), torch.randn(96, 200, generator=g).cuda()
    full = torch.empty(150, 96, device="cuda"); cu.linear(a, w, None, full)
    for lo, hi in ((0, 1), (3, 12), (100, 117), (64, 150)):
        part = torch.empty(hi - lo, 96, device="cuda")
        cu.linear(a[lo:hi].contiguous(), w, None, part)
        assert torch.equal(part, full[lo:hi])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("Hq,Hkv,hd,bs", [(4, 2, 16, 4), (3, 1, 32, 8), (5, 5, 48, 4), (14, 2, 64, 16), (8, 2, 128, 16)])
def test_rope_kv_write(dtype, Hq, Hkv, hd, bs):
    cu, pl = ops_pair(dtype)
    g = torch.Generator().manual_seed(hd)
    max_len, mb, pages = 64, 64 // bs, 40
    ang = torch.rand(max_len, hd // 2, generator=g) * 6
    cos, sin = torch.cos(ang), torch.sin(ang)
    # two requests: rows 0..5 of request 0 at positions 9..14, a padding row, rows of request 1 at positions 0..3
    pos = list(range(9, 15)) + [0] + list(range(0, 4))
    seq_row = [0] * 6 + [-1] + [1] * 4
    perm = torch.randperm(pages, generator=g).tolist()
    table = [perm[:mb], perm[mb:2 * mb]]
    n = len(pos)
    qkv = torch.randn(n, (Hq + 2 * Hkv) * hd, generator=g)
    meta_c, meta_p = Meta(pos, seq_row, table, "cuda"), Meta(pos, seq_row, table, "cpu")
    cc, cp = make_cache(pages, Hkv, bs, hd, DT[dtype], "cuda"), make_cache(pages, Hkv, bs, hd, DT[dtype], "cpu")
    q, qp = torch.empty(n, Hq * hd, dtype=DT[dtype], device="cuda"), torch.empty(n, Hq * hd, dtype=DT[dtype])
    cu.rope_kv_write(qkv.cuda(), cos.cuda(), sin.cuda(), meta_c, cc, q, Hq, Hkv, hd)
    pl.rope_kv_write(qkv, cos, sin, meta_p, cp, qp, Hq, Hkv, hd)
    close(q, qp, dtype, steps=1.01)
    close(cc.pool, cp.pool, dtype, steps=1.01)
    assert int((cc.pool != 0).any(-1).sum()) == int((cp.pool != 0).any(-1).sum()), "only the step's slots are written"
    # write=False stores nothing
    cc2 = make_cache(pages, Hkv, bs, hd, DT[dtype], "cuda", write=False)
    cu.rope_kv_write(qkv.cuda(), cos.cuda(), sin.cuda(), meta_c, cc2, q, Hq, Hkv, hd)
    assert float(cc2.pool.float().abs().max()) == 0.0
    cu.check_errors()


def fill_cache(cache, table, lengths, g, scale=1.0):
    """Random keys and values for positions [0, lengths[r]) of every request r, through its block table."""
    bs = cache.page_size
    hkv, hd = cache.keys.shape[1], cache.keys.shape[3]
    for r, L in enumerate(lengths):
        for p in range(L):
            page = table[r][p // bs]
            cache.keys[page, :, p % bs] = (torch.randn(hkv, hd, generator=g) * scale).to(cache.keys.dtype)
            cache.values[page, :, p % bs] = torch.randn(hkv, hd, generator=g).to(cache.values.dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("Hq,Hkv,hd,bs,window", [(4, 2, 16, 4, 0), (3, 1, 32, 8, 0), (5, 5, 48, 4, 12), (14, 2, 64, 16, 0),
                                                  (8, 2, 128, 16, 37), (20, 2, 80, 16, 0), (2, 1, 256, 8, 0),
                                                  # more query heads per kv head than one block takes (32), an odd remainder,
                                                  # and head sizes beyond 256
                                                  (70, 2, 16, 8, 0), (33, 1, 48, 4, 20), (2, 2, 384, 16, 0), (3, 1, 512, 8, 0)])
def test_paged_attention(dtype, Hq, Hkv, hd, bs, window):
    cu, pl = ops_pair(dtype)
    g = torch.Generator().manual_seed(Hq * hd + window)
    lengths = [150, 33, 1, 64]
    mb, pages = -(-160 // bs), 4 * -(-160 // bs) + 3
    perm = torch.randperm(pages, generator=g).tolist()
    table = [perm[r * mb:(r + 1) * mb] for r in range(4)]
    cp = make_cache(pages, Hkv, bs, hd, DT[dtype], "cpu")
    fill_cache(cp, table, lengths, g)
    cc = make_cache(pages, Hkv, bs, hd, DT[dtype], "cuda")
    cc.pool.copy_(cp.pool)
    # rows: a portion of request 0 (positions 140..149), one token of request 1, padding, request 2's only token,
    # a portion of request 3 that crosses pages
    pos = list(range(140, 150)) + [32] + [0] + [0] + list(range(50, 64))
    seq_row = [0] * 10 + [1] + [-1] + [2] + [3] * 14
    n = len(pos)
    q = torch.randn(n, Hq * hd, generator=g).to(DT[dtype])
    o, op = torch.empty(n, Hq * hd, dtype=DT[dtype], device="cuda"), torch.empty(n, Hq * hd, dtype=DT[dtype])
    scale = hd ** -0.5
    cu.paged_attention(q.cuda(), cc, Meta(pos, seq_row, table, "cuda"), o, Hq, Hkv, hd, scale, window)
    pl.paged_attention(q, cp, Meta(pos, seq_row, table, "cpu"), op, Hq, Hkv, hd, scale, window)
    close(o, op, dtype)
    assert float(o[11].float().abs().max()) == 0.0, "a padding row gives zeros"
    cu.check_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [0, 100])
def test_paged_attention_finds_a_far_key(dtype, window):
    """One key among hundreds is made to stand out (it is a large multiple of the query); the output must be that key's
    value. With a window the key sits on the window's first position, and one position earlier it must be invisible."""
    cu, _ = ops_pair(dtype)
    Hq, Hkv, hd, bs = 4, 2, 64, 16
    g = torch.Generator().manual_seed(7)
    L = 700
    mb = -(-L // bs)
    perm = torch.randperm(mb + 5, generator=g).tolist()
    table = [perm[:mb]]
    cp = make_cache(mb + 5, Hkv, bs, hd, DT[dtype], "cpu")
    fill_cache(cp, table, [L], g, scale=0.1)
    q = torch.randn(1, Hq * hd, generator=g)
    q = (q / q.view(Hq, hd).norm(dim=-1).repeat_interleave(hd)).to(DT[dtype])
    p = L - 1
    for far, visible in (((p - window + 1) if window else 3, True), ((p - window) if window else None, False)):
        if far is None:
            continue
        cc = make_cache(mb + 5, Hkv, bs, hd, DT[dtype], "cuda")
        pool = cp.pool.clone()
        page, off = table[0][far // bs], far % bs
        for kvh in range(Hkv):   # the key of kv head kvh = 60 x the query of its first query head
            pool[page, 0, kvh, off] = (q.view(Hq, hd)[kvh * (Hq // Hkv)].float() * 60).to(DT[dtype])
            pool[page, 1, kvh, off] = 5.0
        cc.pool.copy_(pool)
        o = torch.empty(1, Hq * hd, dtype=DT[dtype], device="cuda")
        cu.paged_attention(q.cuda(), cc, Meta([p], [0], table, "cuda"), o, Hq, Hkv, hd, 1.0, window)
        first_heads = o.view(Hq, hd)[::Hq // Hkv].float().cpu()
        if visible:
            assert (first_heads - 5.0).abs().max() < 0.05, f"the far key at {far} was not found: {first_heads[:, :3]}"
        else:
            assert first_heads.abs().max() < 2.0, f"a key before the window at {far} was seen: {first_heads[:, :3]}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_swiglu(dtype):
    cu, pl = ops_pair(dtype)
    g = torch.Generator().manual_seed(2)
    gu = (torch.randn(23, 2 * 176, generator=g) * 4).to(DT[dtype])
    o, op = torch.empty(23, 176, dtype=DT[dtype], device="cuda"), torch.empty(23, 176, dtype=DT[dtype])
    cu.swiglu(gu.cuda(), o)
    pl.swiglu(gu, op)
    close(o, op, dtype, steps=1.01)


def test_argmax_ties_and_nan():
    cu, _ = ops_pair("float32")
    g = torch.Generator().manual_seed(3)
    a = torch.randn(6, 5003, generator=g)
    a[1, 100] = a[1, 4000] = 9.0           # a tie: the first index wins
    a[2, 77] = float("nan"); a[2, 3] = 50  # a NaN is the maximum
    a[3, 4999] = float("nan"); a[3, 200] = float("nan")
    a[4] = -float("inf")
    a[5, 5002] = 30.0
    out = torch.empty(6, dtype=torch.int32, device="cuda")
    cu.argmax(a.cuda(), out)
    assert out.cpu().tolist() == np.argmax(a.numpy(), -1).tolist() == [int(a[0].argmax()), 100, 77, 200, 0, 5002]


def test_sample_matches_the_host_rule():
    cu, pl = ops_pair("float32")
    g = torch.Generator().manual_seed(4)
    R, V = 64, 1511
    lg = torch.randn(R, V, generator=g) * 3
    temp = torch.full((R,), 0.8); temp[5] = 0.0; temp[6] = 2.5
    u = torch.rand(R, generator=g, dtype=torch.float64); u[7] = 0.0; u[8] = 1.0 - 2.0 ** -53
    out, outp = torch.empty(R, dtype=torch.int32, device="cuda"), torch.empty(R, dtype=torch.int32)
    cu.sample(lg.cuda(), temp.cuda(), u.cuda(), out)
    pl.sample(lg, temp, u, outp)
    assert out.cpu().tolist() == outp.tolist()
    assert int(out[5]) == int(lg[5].argmax())


@pytest.mark.parametrize("V", [1511, 50257])
def test_sample_filtered_matches_the_host_rule(V):
    """Top-k and top-p on the device against the plain filters: every mix of the two, rows that are greedy, logits on a
    coarse grid (so that equal values sit at both thresholds), masked tokens, and draws at both ends."""
    cu, pl = ops_pair("float32")
    g = torch.Generator().manual_seed(9)
    R = 40
    lg = torch.randn(R, V, generator=g) * 3
    lg[8:16] = (lg[8:16] * 2).round() / 2              # many equal values
    lg[16:20] = (lg[16:20] / 4).round()                # a handful of distinct values: long runs of equals at a threshold
    lg[20, ::3] = -float("inf")
    lg[21] = 0.0                                       # all equal
    lg[22, 100] = 60.0                                 # one token holds all the mass
    temp = torch.full((R,), 0.8); temp[5] = 0.0; temp[6] = 2.5; temp[24:32] = 1.7
    top_k = torch.zeros(R, dtype=torch.int32); top_p = torch.ones(R)
    ks = [0, 1, 2, 7, 50, 300, V - 1, V, V + 5]
    ps = [1.0, 0.999, 0.9, 0.5, 0.1, 1e-6]
    for r in range(R):
        top_k[r] = ks[r % len(ks)]
        top_p[r] = ps[(r // 2) % len(ps)]
    u = torch.rand(R, generator=g, dtype=torch.float64); u[7] = 0.0; u[9] = 1.0 - 2.0 ** -53; u[17] = 0.0; u[18] = 1.0 - 2.0 ** -53
    out, outp = torch.empty(R, dtype=torch.int32, device="cuda"), torch.empty(R, dtype=torch.int32)
    cu.sample_filtered(lg.cuda(), temp.cuda(), top_k.cuda(), top_p.cuda(), u.cuda(), out)
    pl.sample_filtered(lg, temp, top_k, top_p, u, outp)
    assert out.cpu().tolist() == outp.tolist()
    again = torch.empty_like(out)
    cu.sample_filtered(lg.cuda(), temp.cuda(), top_k.cuda(), top_p.cuda(), u.cuda(), again)
    assert torch.equal(out, again)
    # without filters it is the plain sampling kernel
    plain = torch.empty_like(out)
    cu.sample(lg.cuda(), temp.cuda(), u.cuda(), plain)
    cu.sample_filtered(lg.cuda(), temp.cuda(), torch.zeros_like(top_k).cuda(), torch.ones(R).cuda(), u.cuda(), again)
    assert torch.equal(plain, again)


def test_refusals():
    cu, _ = ops_pair("float32")
    from fusezap_core_b200.kernels.table import KernelError
    with pytest.raises(ValueError, match="multiple of 16"):
        cu.check_attention(4, 2, 24)
    with pytest.raises(ValueError, match="not supported"):
        cu.check_attention(8, 2, 528)
    with pytest.raises(ValueError, match="not supported"):
        cu.check_attention(7, 2, 64)
    cu.check_attention(66, 2, 64)      # any group size
    with pytest.raises(KernelError, match="CUDA tensors only"):
        cu.swiglu(torch.zeros(2, 8), torch.zeros(2, 4))
