"""The tcgen05 / TMA matrix product alone, against a plain float32 product of the same bfloat16 operands: few rows
(swapped operands, with and without split K), many rows, ragged edges in every dimension, bias, both output dtypes."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def run(M, N, K, out_dtype, bias, seed=0):
    from fusezap_core_b200.kernels import cuda_ops
    ops = cuda_ops("bfloat16")
    assert ops.use_tensor_cores
    g = torch.Generator().manual_seed(seed + M + 3 * N + 7 * K)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w = torch.randn(N, K, generator=g).to(torch.bfloat16).cuda()
    b = torch.randn(N, generator=g).cuda() if bias else None
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device="cuda")
    before = ops.launches
    ops.linear(a, w, b, out)
    ops.check_errors()
    assert ops.launches == before + 1
    ref = a.double() @ w.double().T
    if b is not None:
        ref = ref + b.double()
    return out, ref


def check(out, ref, K):
    out, ref = out.double().cpu(), ref.cpu()
    assert torch.isfinite(out).all(), "unwritten or non-finite outputs"
    scale = float(ref.abs().max())
    err = float((out - ref).abs().max())
    return err, scale


@pytest.mark.parametrize("M", [1, 8, 16, 17, 33, 64, 100, 128])
@pytest.mark.parametrize("N,K", [(1000, 4096), (512, 4096), (128, 64), (48, 80), (6144, 512), (384, 96)])
def test_few_rows(M, N, K):
    for out_dtype, bias in ((torch.float32, False), (torch.bfloat16, True)):
        out, ref = run(M, N, K, out_dtype, bias)
        err, scale = check(out, ref, K)
        lim = 1e-4 * scale if out_dtype == torch.float32 else 2.0 ** -8 * scale
        assert err <= lim, f"M={M} N={N} K={K} {out_dtype}: max |diff| {err:.3e} > {lim:.3e}"


@pytest.mark.parametrize("M,N,K", [(129, 256, 128), (300, 777, 200), (2048, 1024, 512), (257, 64, 4096), (1000, 136, 72),
                                   (384, 96, 96),
                                   # fewer tiles than SMs, or a partial last round, with a long K
                                   (256, 4096, 4096), (512, 6144, 4096), (200, 1000, 8192), (2048, 4096, 4096), (640, 4096, 1024),
                                   (512, 8192, 512),      # tiles 160, 192, 160, 256, 160 and 224 columns wide
                                   # few tiles and a long K: the K range of a tile is cut over a cluster of 2 to 8 CTAs
                                   (300, 4096, 14336), (384, 777, 1024), (130, 256, 8200), (256, 6144, 4096),
                                   # many rounds and a short K
                                   (150, 151936, 896)])
def test_many_rows(M, N, K):
    for out_dtype, bias in ((torch.float32, True), (torch.bfloat16, False)):
        out, ref = run(M, N, K, out_dtype, bias)
        err, scale = check(out, ref, K)
        lim = 1e-4 * scale if out_dtype == torch.float32 else 2.0 ** -8 * scale
        assert err <= lim, f"M={M} N={N} K={K} {out_dtype}: max |diff| {err:.3e} > {lim:.3e}"


@pytest.fixture
def rows_mode():
    """Forces one of the many-token kernels (1: one SM per tile, 2: a pair of SMs per 256 x 256 tile) and puts the rule
    back afterwards."""
    from fusezap_core_b200.kernels import cuda_ops
    tc = cuda_ops("bfloat16").tc
    yield tc.fz_gemm_tc_rows_mode
    tc.fz_gemm_tc_rows_mode(0)


@pytest.mark.parametrize("M,N,K", [(129, 256, 64), (256, 256, 128), (257, 300, 72), (300, 777, 200), (1000, 4096, 1024),
                                   (2048, 1024, 512), (640, 6144, 4096), (1153, 5000, 264),
                                   (150, 151936, 896),      # one pair of SMs walks more tiles than it has accumulators
                                   # few tiles and a long K: pairs of SMs in clusters of 4 that cut K in two
                                   (256, 6144, 4096), (512, 4096, 14336), (512, 4096, 4096), (200, 1000, 1100), (130, 300, 1032)])
def test_many_rows_on_pairs_of_sms(M, N, K, rows_mode):
    """The two-SM kernels (each CTA of a pair holds half of the tile's token rows and half of its features; with K cut
    over the cluster or not) against float64, with ragged edges in every dimension and token rows that leave the pair's
    second half empty; and bit for bit against the one-SM kernels where K is cut into as many pieces (the sums over K
    then have the same order)."""
    from fusezap_core_b200.kernels import cuda_ops
    tc = cuda_ops("bfloat16").tc
    rows_mode(2)
    same_order = tc.fz_gemm_tc_rows_pair_splits(M, N, K) in (tc.fz_gemm_tc_rows_splits(M, N, K), 1) and \
        (tc.fz_gemm_tc_rows_pair_splits(M, N, K) > 1 or tc.fz_gemm_tc_rows_splits(M, N, K) == 1)
    outs = {}
    for mode in (1, 2):
        rows_mode(mode)
        for out_dtype, bias in ((torch.float32, True), (torch.bfloat16, False)):
            out, ref = run(M, N, K, out_dtype, bias)
            err, scale = check(out, ref, K)
            lim = 1e-4 * scale if out_dtype == torch.float32 else 2.0 ** -8 * scale
            assert err <= lim, f"mode {mode} M={M} N={N} K={K} {out_dtype}: max |diff| {err:.3e} > {lim:.3e}"
            outs[mode, out_dtype] = out
    for out_dtype in (torch.float32, torch.bfloat16):
        if same_order:
            assert torch.equal(outs[1, out_dtype], outs[2, out_dtype]), f"{out_dtype}: the two kernels differ"


def test_which_products_go_to_pairs_of_sms():
    from fusezap_core_b200.kernels import cuda_ops
    tc = cuda_ops("bfloat16").tc
    tc.fz_gemm_tc_rows_mode(0)
    for M, N, K in ((2048, 6144, 4096), (2048, 4096, 14336), (1024, 28672, 4096), (512, 28672, 4096), (256, 28672, 4096),
                    (1200, 4096, 4096)):
        assert tc.fz_gemm_tc_rows_pairs(M, N, K) == 1, (M, N, K)
    # few rows, an odd count of 128-row tiles below nine, narrow outputs, or too few tiles for half a round
    for M, N, K in ((128, 4096, 4096), (384, 28672, 4096), (640, 28672, 4096), (2048, 128, 4096), (256, 1024, 4096)):
        assert tc.fz_gemm_tc_rows_pairs(M, N, K) == 0, (M, N, K)


def test_which_products_are_cut_along_k():
    from fusezap_core_b200.kernels import cuda_ops
    tc = cuda_ops("bfloat16").tc
    tc.fz_gemm_tc_rows_mode(0)
    # on pairs of SMs where the 128-row tiles come in an even count and the clusters stay within 128 CTAs
    assert tc.fz_gemm_tc_rows_pair_splits(256, 6144, 4096) == 2 and tc.fz_gemm_tc_rows_pair_splits(512, 4096, 14336) == 2
    assert tc.fz_gemm_tc_rows_pair_splits(512, 4096, 4096) == 2
    for M, N, K in ((384, 4096, 14336), (2048, 4096, 4096), (256, 4096, 256), (128, 4096, 4096), (256, 4096, 14336),
                    (200, 1000, 8192)):
        assert tc.fz_gemm_tc_rows_pair_splits(M, N, K) == 1, (M, N, K)
    assert tc.fz_gemm_tc_rows_splits(256, 6144, 4096) == 2 and tc.fz_gemm_tc_rows_splits(256, 4096, 14336) == 4
    assert tc.fz_gemm_tc_rows_splits(200, 1000, 8192) == 8 and tc.fz_gemm_tc_rows_splits(384, 777, 1024) == 2
    for M, N, K in ((2048, 4096, 4096), (512, 6144, 4096), (128, 4096, 4096), (256, 4096, 256), (256, 128, 4096)):
        assert tc.fz_gemm_tc_rows_splits(M, N, K) == 1, (M, N, K)


def test_a_row_does_not_depend_on_the_other_rows():
    """Few rows: the same row gives the same bits alone and among 8, 16 or 64 rows (the split of K depends on N and K
    only, and the sum over the splits has one order)."""
    from fusezap_core_b200.kernels import cuda_ops
    ops = cuda_ops("bfloat16")
    g = torch.Generator().manual_seed(5)
    a = torch.randn(64, 2048, generator=g).to(torch.bfloat16).cuda()
    w = torch.randn(640, 2048, generator=g).to(torch.bfloat16).cuda()
    full = torch.empty(64, 640, device="cuda"); ops.linear(a, w, None, full)
    for rows in (1, 8, 16, 40):
        part = torch.empty(rows, 640, device="cuda")
        ops.linear(a[:rows].contiguous(), w, None, part)
        assert torch.equal(part, full[:rows]), f"{rows} rows"
    again = torch.empty(64, 640, device="cuda"); ops.linear(a, w, None, again)
    assert torch.equal(again, full), "split-K sums are deterministic"
    ops.check_errors()


def test_refused_shapes_fall_back_to_the_plain_kernel():
    from fusezap_core_b200.kernels import cuda_ops
    ops = cuda_ops("bfloat16")
    g = torch.Generator().manual_seed(6)
    a = torch.randn(5, 36, generator=g).to(torch.bfloat16).cuda()      # K = 36 is no multiple of 8
    w = torch.randn(20, 36, generator=g).to(torch.bfloat16).cuda()
    out = torch.empty(5, 20, device="cuda")
    ops.linear(a, w, None, out)
    assert float((out.double() - a.double() @ w.double().T).abs().max()) < 1e-3


@pytest.mark.parametrize("M", [1, 8, 40, 128, 129, 700])
@pytest.mark.parametrize("I,K", [(128, 64), (448, 96), (4864, 896), (1024, 4096)])
@pytest.mark.parametrize("mode", [1, 2])
def test_fused_gate_up_swiglu(M, I, K, mode, rows_mode):
    """The fused product + SwiGLU against silu(x.gate^T + bg) * (x.up^T + bu) in float64, in both modes (few rows: with
    and without a split of K; many rows: persistent tiles on one SM or on a pair)."""
    from fusezap_core_b200.kernels import cuda_ops
    ops = cuda_ops("bfloat16")
    if mode == 2 and M <= 128:
        pytest.skip("few rows never go to the many-token kernels")
    rows_mode(mode)
    g = torch.Generator().manual_seed(M + I + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    wg = (torch.randn(I, K, generator=g) * K ** -0.5).to(torch.bfloat16).cuda()
    wu = (torch.randn(I, K, generator=g) * K ** -0.5).to(torch.bfloat16).cuda()
    for bias in (False, True):
        bg = torch.randn(I, generator=g).cuda() if bias else None
        bu = torch.randn(I, generator=g).cuda() if bias else None
        packed = ops.pack_gate_up(wg, wu, bg, bu)
        assert packed is not None
        out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device="cuda")
        ops.linear_swiglu(x, packed, out)
        ops.check_errors()
        gg = x.double() @ wg.double().T + (bg.double() if bias else 0)
        uu = x.double() @ wu.double().T + (bu.double() if bias else 0)
        ref = gg / (1 + torch.exp(-gg)) * uu
        err = float((out.double() - ref).abs().max())
        lim = 2.0 ** -8 * float(ref.abs().max()) * 1.01
        assert torch.isfinite(out.float()).all() and err <= lim, f"M={M} I={I} K={K} bias={bias}: {err:.3e} > {lim:.3e}"
    assert ops.pack_gate_up(wg[:100], wu[:100]) is None, "I must be a multiple of 64"


@pytest.mark.parametrize("Hq,Hkv,hd,K,bs", [(32, 8, 128, 4096, 16), (14, 2, 64, 896, 8), (3, 1, 64, 128, 5), (5, 5, 32, 200, 16),
                                            (2, 1, 128, 64, 3)])
@pytest.mark.parametrize("M", [1, 8, 19, 32])
def test_qkv_product_with_rotation_and_cache_write(Hq, Hkv, hd, K, bs, M):
    """The q/k/v product that ends in the rotation and the cache write gives the bits of the product followed by the
    rotation kernel: q, and every slot of the key and value pools (written ones and untouched ones); with a bias, a
    padding row, rows of several requests at scattered positions, whole heads that straddle nothing (hd divides 128)
    and a last tile that is not full; and it leaves the pool alone when the layer does not write its cache."""
    from types import SimpleNamespace
    from fusezap_core_b200.kernels import cuda_ops
    from test_kernels_gpu import Meta, make_cache
    ops = cuda_ops("bfloat16")
    g = torch.Generator().manual_seed(Hq * 7 + hd + M)
    N = (Hq + 2 * Hkv) * hd
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K, generator=g) * K ** -0.5).to(torch.bfloat16).cuda()
    b = torch.randn(N, generator=g).cuda()
    max_len = 700
    ang = torch.rand(max_len, hd // 2, generator=g) * 6.28
    cos, sin = torch.cos(ang).cuda(), torch.sin(ang).cuda()
    n_req = 3
    mb = -(-max_len // bs)
    perm = torch.randperm(n_req * mb + 2, generator=g).tolist()
    table = [perm[r * mb:(r + 1) * mb] for r in range(n_req)]
    pos, seq = [], []
    used = set()
    for i in range(M):
        r = i % n_req
        p = int(torch.randint(0, max_len, (1,), generator=g))
        while (r, p) in used:
            p = (p + 1) % max_len
        used.add((r, p)); pos.append(p); seq.append(r)
    if M > 2:
        seq[M // 2] = -1
    meta = Meta(pos, seq, table, "cuda")
    for write in (True, False):
        res = []
        for fused in (True, False):
            cache = make_cache(n_req * mb + 2, Hkv, bs, hd, torch.bfloat16, "cuda", write=write)
            cache.pool.copy_(torch.randn(cache.pool.shape, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16))
            q = torch.full((M, Hq * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
            if fused:
                assert ops.linear_rope_kv_write(a, w, b, cos, sin, meta, cache, q, Hq, Hkv, hd)
            else:
                qkv = torch.empty(M, N, device="cuda")
                ops.linear(a, w, b, qkv)
                ops.rope_kv_write(qkv, cos, sin, meta, cache, q, Hq, Hkv, hd)
            ops.check_errors()
            res.append((q.clone(), cache.pool.clone()))
        assert torch.isfinite(res[0][0].float()).all()
        assert torch.equal(res[0][0], res[1][0]), f"write={write}: q differs"
        assert torch.equal(res[0][1], res[1][1]), f"write={write}: the pools differ"
    # sizes the fused kernel does not take are refused, not computed
    q = torch.empty(200, Hq * hd, dtype=torch.bfloat16, device="cuda")
    big = torch.randn(200, K, generator=g).to(torch.bfloat16).cuda()
    assert ops.linear_rope_kv_write(big, w, b, cos, sin, meta, cache, q, Hq, Hkv, hd) is False


@pytest.mark.parametrize("M,N,K", [(1, 20000, 256), (8, 33333, 128), (37, 17000, 64), (128, 16512, 72)])
def test_product_that_keeps_only_the_largest_of_each_row(M, N, K):
    """`linear_argmax` gives the ids that `argmax` finds in the logits `linear` writes, with the numpy rule for ties (the
    lower index) and NaN (a NaN wins), a bias, a ragged last tile; sizes whose K is split are refused."""
    from fusezap_core_b200.kernels import cuda_ops
    ops = cuda_ops("bfloat16")
    g = torch.Generator().manual_seed(M + N)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w = torch.randn(N, K, generator=g).to(torch.bfloat16).cuda()
    w[N - 1] = w[5]                      # equal logits at 5 and N - 1 in every row: the lower index must win where they are the maximum
    w[N // 2] = w[5]
    a[0] = 0                             # a row of all-equal logits
    b = (torch.randn(N, generator=g) * 0.01).cuda()
    b[N - 1] = b[5]; b[N // 2] = b[5]
    for bias in (None, b):
        logits = torch.empty(M, N, device="cuda")
        ops.linear(a, w, bias, logits)
        want = torch.empty(M, dtype=torch.int32, device="cuda")
        ops.argmax(logits, want)
        got = torch.full((M,), -1, dtype=torch.int32, device="cuda")
        assert ops.linear_argmax(a, w, bias, got)
        ops.check_errors()
        assert torch.equal(got, want), (got.tolist(), want.tolist())
        assert bias is not None or int(got[0]) == 0
    if M > 1:
        a2 = a.clone(); a2[1, 3] = float("nan")            # a NaN activation makes the whole row NaN: index 0
        got = torch.full((M,), -1, dtype=torch.int32, device="cuda")
        assert ops.linear_argmax(a2, w, None, got) and int(got[1]) == 0
    # few tiles and a long K: the product would be split along K; refused, the caller writes logits and uses `argmax`
    a3 = torch.randn(M, 4096, generator=g).to(torch.bfloat16).cuda()
    w3 = torch.randn(1024, 4096, generator=g).to(torch.bfloat16).cuda()
    assert ops.linear_argmax(a3, w3, None, got) is False
