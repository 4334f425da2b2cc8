"""The tensor-core attention kernels alone (bf16 cache): the split decode kernel with its combine, and the tile
prefill kernel, against the plain reference, at head sizes 64 and 128, groups of 1 to 16 query heads per kv head, long
contexts across several key partitions, portions that span several 64-row tiles, windows, odd page sizes."""
import pytest
import torch

from plain_ops import PlainOps
from test_kernels_gpu import Meta, fill_cache, make_cache

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def run_both(Hq, Hkv, hd, bs, window, lengths, rows, seed=0, prefill_mode=0):
    """rows: list of (request, first position, count). Returns (cuda out, plain out, ops). prefill_mode: which prompt
    kernel takes the long portions (0: chosen by shape, 1: one head per block, 2: two heads per block)."""
    from fusezap_core_b200.kernels import cuda_ops
    cu, pl = cuda_ops("bfloat16"), PlainOps(BF)
    assert cu.use_tensor_cores and cu.tc.fz_attn_decode_check(Hq, Hkv, hd) == 0
    assert cu.tc.fz_attn_prefill_tc_mode(prefill_mode) == 0
    g = torch.Generator().manual_seed(seed + Hq + hd + window)
    mb = -(-max(lengths) // bs)
    pages = mb * len(lengths) + 3
    perm = torch.randperm(pages, generator=g).tolist()
    table = [perm[r * mb:(r + 1) * mb] for r in range(len(lengths))]
    cp = make_cache(pages, Hkv, bs, hd, BF, "cpu")
    fill_cache(cp, table, lengths, g)
    cc = make_cache(pages, Hkv, bs, hd, BF, "cuda")
    cc.pool.copy_(cp.pool)
    pos, seq_row = [], []
    for req, p0, cnt in rows:
        pos += list(range(p0, p0 + cnt)); seq_row += [req] * cnt
    n = len(pos)
    q = torch.randn(n, Hq * hd, generator=g).to(BF)
    o, op = torch.full((n, Hq * hd), float("nan"), dtype=BF, device="cuda"), torch.empty(n, Hq * hd, dtype=BF)
    scale = hd ** -0.5
    # (tiles are cut along the keys only where the tcgen05 prompt kernel runs: pages that TMA can box)
    meta = Meta(pos, seq_row, table, "cuda", cut_keys=bs == 8 or bs % 16 == 0, heads=Hq,
                items=Hkv * ((Hq // Hkv + 1) // 2) if hd == 128 else Hq)
    try:
        cu.paged_attention(q.cuda(), cc, meta, o, Hq, Hkv, hd, scale, window)
    finally:
        cu.tc.fz_attn_prefill_tc_mode(0)
    pl.paged_attention(q, cp, Meta(pos, seq_row, table, "cpu"), op, Hq, Hkv, hd, scale, window)
    cu.check_errors()
    run_both.last_plan = meta.plan
    return o.float().cpu(), op.float(), seq_row


def close(o, op, what):
    assert torch.isfinite(o).all(), f"{what}: unwritten or non-finite rows {torch.where(~torch.isfinite(o).all(-1))[0][:8].tolist()}"
    err = (o - op).abs().max(-1).values
    tol = 2.0 ** -7 * max(float(op.abs().max()), 1e-3)      # two bf16 steps: P is rounded to bf16 before P.V
    bad = torch.where(err > tol)[0]
    assert len(bad) == 0, f"{what}: rows {bad[:8].tolist()} differ by {float(err.max()):.3e} > {tol:.3e}"


@pytest.mark.parametrize("Hq,Hkv,hd", [(8, 2, 128), (14, 2, 64)])
def test_decode_rows_do_not_depend_on_the_batch(Hq, Hkv, hd):
    """The same three decoded tokens alone and among 33 others: the kernels size their blocks by the number of rows (the
    combine kernel takes blocks of 256 threads while there are fewer blocks than SMs), and every bit of a row must
    stay what it was."""
    g = torch.Generator().manual_seed(5)
    lengths = [4300, 777, 2050] + torch.randint(40, 3000, (33,), generator=g).tolist()
    rows = [(r, n - 1, 1) for r, n in enumerate(lengths)]
    few, ref, _ = run_both(Hq, Hkv, hd, 16, 0, lengths, rows[:3], seed=11)
    many, _, _ = run_both(Hq, Hkv, hd, 16, 0, lengths, rows, seed=11)
    close(few, ref, "three rows")
    assert torch.equal(few, many[:3]), "a row's bits changed with the batch"


@pytest.mark.parametrize("Hq,Hkv,hd", [(4, 1, 128), (14, 2, 64), (8, 8, 64), (16, 1, 128), (10, 2, 128), (3, 3, 64)])
@pytest.mark.parametrize("bs,window", [(16, 0), (8, 300), (5, 0), (64, 0), (48, 200)])
def test_decode_rows_at_long_contexts(Hq, Hkv, hd, bs, window):
    lengths = [1100, 257, 1, 640]
    # single tokens at the ends of partitions and tiles, the first token, and short portions (below 8 rows)
    rows = [(0, 1099, 1), (1, 255, 2), (2, 0, 1), (3, 511, 1), (3, 512, 1), (0, 62, 3), (3, 633, 7)]
    o, op, _ = run_both(Hq, Hkv, hd, bs, window, lengths, rows)
    close(o, op, "decode")


@pytest.mark.parametrize("Hq,Hkv,hd,bs", [(8, 2, 128, 16), (6, 3, 64, 8), (4, 2, 128, 32)])
@pytest.mark.parametrize("window", [0, 700])
def test_decode_rows_past_4096_keys(Hq, Hkv, hd, bs, window):
    """Beyond key 4096 the key axis is cut into units of 256 instead of 64: rows at both sides of the change, at the
    edges of the larger units, and with a window that begins among the small units and ends among the large ones."""
    lengths = [5000, 4400, 4097]
    rows = [(0, 4999, 1), (0, 4095, 1), (0, 4096, 1), (1, 4351, 1), (1, 4352, 2), (2, 4096, 1), (1, 100, 1), (0, 4700, 5)]
    o, op, _ = run_both(Hq, Hkv, hd, bs, window, lengths, rows)
    close(o, op, "decode past 4096")


@pytest.mark.parametrize("mode", [1, 2])
@pytest.mark.parametrize("Hq,Hkv,hd", [(4, 1, 128), (14, 2, 64), (8, 8, 64), (2, 1, 128), (10, 2, 128), (3, 3, 64)])
@pytest.mark.parametrize("bs,window", [(16, 0), (8, 100), (3, 0), (64, 0), (128, 90), (48, 0)])
def test_prefill_portions(Hq, Hkv, hd, bs, window, mode):
    """Both prompt kernels (one head per block, two heads of a kv head per block) on the same inputs: groups of 1, 2, 3,
    4, 5 and 7 query heads per kv head (odd groups leave a block with a single head), both head sizes."""
    lengths = [400, 70, 200, 400, 31]
    # a first portion from position 0 (two tiles), a later portion that continues a request (ragged last tile),
    # a portion of exactly 8 rows, and single tokens beside them (mixed step)
    rows = [(0, 0, 150), (2, 61, 139), (1, 62, 8), (3, 399, 1), (4, 30, 1)]
    o, op, _ = run_both(Hq, Hkv, hd, bs, window, lengths, rows, prefill_mode=mode)
    close(o, op, "prefill")


@pytest.mark.parametrize("Hq,Hkv,hd,window", [(8, 2, 128, 0), (5, 1, 128, 700), (14, 2, 64, 0)])
def test_prefill_kernels_agree_on_long_portions(Hq, Hkv, hd, window):
    """A 1,300-token portion behind 900 cached tokens (eleven key tiles, through the lazy rescaling of the output many
    times) and a second request: the two prompt kernels do the same arithmetic in the same order, so they give the same
    bits, and both follow the plain reference."""
    lengths = [2200, 517]
    rows = [(0, 900, 1300), (1, 0, 517)]
    one, ref, _ = run_both(Hq, Hkv, hd, 16, window, lengths, rows, seed=5, prefill_mode=1)
    two, _, _ = run_both(Hq, Hkv, hd, 16, window, lengths, rows, seed=5, prefill_mode=2)
    close(one, ref, "one head per block")
    close(two, ref, "two heads per block")
    assert torch.equal(one, two)


@pytest.mark.parametrize("mode", [1, 2])
@pytest.mark.parametrize("Hq,Hkv,hd,bs", [(8, 2, 128, 16), (14, 2, 64, 8), (3, 1, 128, 64)])
@pytest.mark.parametrize("window", [0, 1500])
def test_small_portions_behind_long_prefixes(Hq, Hkv, hd, bs, window, mode):
    """Few query tiles with thousands of keys behind them: the plan cuts the tiles along the keys (pieces of at least
    eight key tiles, merged by a second kernel), in both prompt kernels; with a window the first pieces of a tile see no
    key at all. A portion that is not cut and single tokens share the step."""
    lengths = [5000, 3000, 400, 2000, 77]
    rows = [(0, 4700, 300), (1, 2950, 50), (2, 0, 130), (3, 1999, 1), (4, 70, 7)]
    o, op, _ = run_both(Hq, Hkv, hd, bs, window, lengths, rows, seed=3, prefill_mode=mode)
    plan = run_both.last_plan
    assert plan.n_cuts >= 2 and plan.n_pieces >= 6, "the long tiles of this step are cut along the keys"
    close(o, op, "pieces along the keys")


def test_padding_rows_and_row_independence():
    """A padding row gives zeros; a row's bits do not change with the rows around it."""
    Hq, Hkv, hd = 8, 2, 128
    lengths = [700, 300]
    from fusezap_core_b200.kernels import cuda_ops
    cu = cuda_ops("bfloat16")
    g = torch.Generator().manual_seed(3)
    cc = make_cache(80, Hkv, 16, hd, BF, "cuda")
    table = [list(range(0, 44)), list(range(44, 63)) + [-1] * 25]
    cp = make_cache(80, Hkv, 16, hd, BF, "cpu")
    fill_cache(cp, table, lengths, g)
    cc.pool.copy_(cp.pool)
    q = torch.randn(42, Hq * hd, generator=g).to(BF).cuda()
    pos = [699] + list(range(100, 140)) + [0]
    seq = [0] + [1] * 40 + [-1]
    full = torch.empty(42, Hq * hd, dtype=BF, device="cuda")
    cu.paged_attention(q, cc, Meta(pos, seq, table, "cuda"), full, Hq, Hkv, hd, hd ** -0.5, 0)
    assert float(full[41].float().abs().max()) == 0.0
    one = torch.empty(1, Hq * hd, dtype=BF, device="cuda")
    cu.paged_attention(q[:1].contiguous(), cc, Meta([699], [0], table, "cuda"), one, Hq, Hkv, hd, hd ** -0.5, 0)
    assert torch.equal(one[0], full[0])
    part = torch.empty(40, Hq * hd, dtype=BF, device="cuda")
    cu.paged_attention(q[1:41].contiguous(), cc, Meta(list(range(100, 140)), [1] * 40, table, "cuda"), part, Hq, Hkv, hd, hd ** -0.5, 0)
    assert torch.equal(part, full[1:41])


@pytest.mark.parametrize("Hq,Hkv,hd", [(8, 2, 128), (12, 1, 64)])
def test_a_row_alone_and_among_hundreds(Hq, Hkv, hd):
    """With few rows every 64-key unit of a row is computed by another warp and the combine kernel merges them; with
    hundreds of rows a warp computes whole 256-key blocks and merges their units itself. Both give the same bits."""
    from fusezap_core_b200.kernels import cuda_ops
    cu = cuda_ops("bfloat16")
    g = torch.Generator().manual_seed(11)
    lengths = [1500, 900, 333]
    bs = 16
    mb = -(-max(lengths) // bs)
    table = [list(range(r * mb, (r + 1) * mb)) for r in range(3)]
    cp = make_cache(3 * mb, Hkv, bs, hd, BF, "cpu")
    fill_cache(cp, table, lengths, g)
    cc = make_cache(3 * mb, Hkv, bs, hd, BF, "cuda")
    cc.pool.copy_(cp.pool)
    pos = [1499, 899, 332] + [int(x) for x in torch.randint(200, 1500, (400,), generator=g)]
    seq = [0, 1, 2] + [0] * 400
    q = torch.randn(len(pos), Hq * hd, generator=g).to(BF).cuda()
    q[3:] = q[0]          # the crowd asks request 0 at other positions
    many = torch.empty(len(pos), Hq * hd, dtype=BF, device="cuda")
    # short portions only (no run of 8 consecutive positions): every row goes through the split kernel
    cu.paged_attention(q, cc, Meta(pos, seq, table, "cuda"), many, Hq, Hkv, hd, hd ** -0.5, 0)
    for i in range(3):
        one = torch.empty(1, Hq * hd, dtype=BF, device="cuda")
        cu.paged_attention(q[i:i + 1].contiguous(), cc, Meta([pos[i]], [seq[i]], table, "cuda"), one, Hq, Hkv, hd, hd ** -0.5, 0)
        assert torch.equal(one[0], many[i]), f"row {i}"
    few = torch.empty(3, Hq * hd, dtype=BF, device="cuda")
    cu.paged_attention(q[:3].contiguous(), cc, Meta(pos[:3], seq[:3], table, "cuda"), few, Hq, Hkv, hd, hd ** -0.5, 0)
    assert torch.equal(few, many[:3])
    cu.check_errors()


@pytest.mark.parametrize("Hq,Hkv,hd,bs", [(8, 2, 128, 16), (14, 2, 64, 8)])
def test_decode_rows_without_tma(Hq, Hkv, hd, bs, monkeypatch):
    """The cp.async variant of the decode kernel (the one page sizes without a TMA box get) on sizes the TMA variant
    normally takes: FZB200_NO_TMA_ATTN selects it."""
    monkeypatch.setenv("FZB200_NO_TMA_ATTN", "1")
    lengths = [1100, 257, 1, 640]
    rows = [(0, 1099, 1), (1, 255, 2), (2, 0, 1), (3, 511, 1), (3, 512, 1), (0, 62, 3), (3, 633, 7)]
    o, op, _ = run_both(Hq, Hkv, hd, bs, 0, lengths, rows)
    close(o, op, "decode without TMA")
    o, op, _ = run_both(Hq, Hkv, hd, bs, 300, lengths, rows)
    close(o, op, "decode without TMA, window")
