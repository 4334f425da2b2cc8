"""Each part of a layer alone on the GPU against the plain implementation's function for that part: position
encoding, norm, mixer (attention over the cache), feed-forward and the block that arranges them."""
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_model
from fusezap_core_b200.cache import CacheManager
from fusezap_core_b200.config import PartSpec
from fusezap_core_b200.engine.step import Portion, StepContext, StepMeta, Workspace
from fusezap_core_b200.parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, LayerCache, build

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def context(dtype, needs, page_size=8, pages=32, max_len=128, rows=128):
    from fusezap_core_b200.kernels import cuda_ops
    ops = cuda_ops(dtype)
    dev = torch.device("cuda:0")
    cache = CacheManager(needs, {}, page_size, pages, 4, max_len, ops.dtype, dev)
    meta = StepMeta(dev, rows, rows, 4, len(cache.groups), cache.max_pages_per_request,
                    ops.step_extra_ints(("attention",), rows, 4))
    ctx = StepContext(ops, Workspace(dev, rows), meta, {}, None)
    return ops, cache, meta, ctx


def tol(dtype, ref, steps=2.0):
    s = float(ref.abs().max())
    return 1e-5 * max(s, 1.0) if dtype == "float32" else steps * 2.0 ** -8 * s


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rmsnorm_part(dtype):
    ops, cache, meta, ctx = context(dtype, {})
    norm = build(NORMS, "norm", PartSpec("rmsnorm", {"size": 72, "eps": 3e-6}))
    assert list(norm.tensors()) == ["weight"] and norm.tensors()["weight"].shape == (72,)
    g = torch.Generator().manual_seed(0)
    w = 1 + 0.1 * torch.randn(72, generator=g)
    norm.bind({"weight": w.cuda()}, ops)
    x, d = torch.randn(9, 72, generator=g), torch.randn(9, 72, generator=g)
    xc = x.clone().cuda()
    h = norm.forward(ctx, xc, d.cuda())
    ref = plain_model.rmsnorm(x + d, w, 3e-6)
    assert torch.equal(xc.cpu(), x + d)
    assert float((h.float().cpu() - ref).abs().max()) <= tol(dtype, ref)
    rows = torch.tensor([4, 0], dtype=torch.int32, device="cuda")
    h2 = norm.forward(ctx, xc, None, rows=rows)
    assert float((h2.float().cpu() - ref[[4, 0]]).abs().max()) <= tol(dtype, ref)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("scaling", [None, {"kind": "linear", "factor": 4.0},
                                     {"kind": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                      "original_max_position_embeddings": 32}])
def test_rotary_part(dtype, scaling):
    hd, Hq, Hkv = 32, 3, 1
    ops, cache, meta, ctx = context(dtype, {0: __import__("fusezap_core_b200.cache", fromlist=["KVNeed"]).KVNeed(Hkv, hd, 0)})
    rope = build(POSITIONS, "position encoding", PartSpec("rope", {"head_dim": hd, "theta": 10000.0, **(scaling or {})}))
    rope.prepare(128, torch.device("cuda:0"))
    hf = None if scaling is None else {("rope_type" if k == "kind" else k): v for k, v in scaling.items()}
    cos, sin = plain_model.rope_tables(hd, 10000.0, hf, 128)
    np.testing.assert_allclose(rope.cos.cpu().numpy(), cos.numpy(), rtol=0, atol=1e-6)
    np.testing.assert_allclose(rope.sin.cpu().numpy(), sin.numpy(), rtol=0, atol=1e-6)
    # rotate rows at positions 40..52 of one request and read the keys back from its pages
    g = torch.Generator().manual_seed(1)
    n, start = 13, 40
    cache.ensure("a", start + n)
    cache.computed["a"] = start
    meta.fill(cache, [Portion("a", [0] * n, [])], [start], ops=ops, needs=("attention",))
    qkv = torch.randn(n, (Hq + 2 * Hkv) * hd, generator=g)
    lc = LayerCache(*cache.groups[0].view(0), group=0, page_size=8, write=True)
    q = torch.empty(n, Hq * hd, dtype=DT[dtype], device="cuda")
    rope.rotate_and_store(ctx, qkv.cuda(), q, lc, Hq, Hkv, hd)
    x = qkv.view(n, Hq + 2 * Hkv, hd)
    ref_q = plain_model.apply_rope(x[:, :Hq], cos[start:start + n], sin[start:start + n]).reshape(n, -1)
    ref_k = plain_model.apply_rope(x[:, Hq:Hq + Hkv], cos[start:start + n], sin[start:start + n])
    assert float((q.float().cpu() - ref_q).abs().max()) <= tol(dtype, ref_q, 1.01)
    table = cache.table(0, "a")
    for i in range(n):
        p = start + i
        got_k = lc.keys[table[p // 8], :, p % 8].float().cpu()
        got_v = lc.values[table[p // 8], :, p % 8].float().cpu()
        assert float((got_k - ref_k[i]).abs().max()) <= tol(dtype, ref_k, 1.01)
        assert float((got_v - x[i, Hq + Hkv:]).abs().max()) <= tol(dtype, x, 1.01)
    ops.check_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("bias", [False, True])
def test_swiglu_part(dtype, bias):
    ops, cache, meta, ctx = context(dtype, {})
    D, I = 72, 200
    ffn = build(FEED_FORWARDS, "feed-forward", PartSpec("swiglu", {"hidden_size": D, "intermediate_size": I}))
    g = torch.Generator().manual_seed(2)
    w = {"mlp.gate_proj.weight": torch.randn(I, D, generator=g) * 0.2, "mlp.up_proj.weight": torch.randn(I, D, generator=g) * 0.2,
         "mlp.down_proj.weight": torch.randn(D, I, generator=g) * 0.2}
    if bias:
        w.update({"mlp.gate_proj.bias": torch.randn(I, generator=g), "mlp.up_proj.bias": torch.randn(I, generator=g),
                  "mlp.down_proj.bias": torch.randn(D, generator=g)})
    w = {k: v.to(DT[dtype]) if v.dim() == 2 else v for k, v in w.items()}
    ffn.bind({k[4:]: v.cuda() for k, v in w.items()}, ops)
    h = torch.randn(11, D, generator=g).to(DT[dtype])
    out = ffn.forward(ctx, h.cuda())
    ref = plain_model.swiglu_mlp(h.float(), w, "", DT[dtype])
    assert out.dtype == torch.float32
    assert float((out.cpu() - ref).abs().max()) <= tol(dtype, ref, 3.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("Hq,Hkv,hd,window,bias", [(4, 2, 16, 0, False), (3, 1, 32, 0, True), (5, 5, 48, 9, True), (8, 2, 64, 20, False)])
def test_attention_part_and_block(dtype, Hq, Hkv, hd, window, bias):
    """The mixer over the cache in two portions (the second reads the first from the pages), then the whole pre-norm
    block, against `plain_model.attention_layer` and `plain_model.layer` on the whole sequence."""
    from fusezap_core_b200.cache import KVNeed
    D, I, T, cut = 80, 136, 37, 21
    ops, cache, meta, ctx = context(dtype, {0: KVNeed(Hkv, hd, window), 1: KVNeed(Hkv, hd, window)})
    g = torch.Generator().manual_seed(Hq * hd)
    mk = lambda *s: (torch.randn(*s, generator=g) * 0.15)
    w = {"self_attn.q_proj.weight": mk(Hq * hd, D), "self_attn.k_proj.weight": mk(Hkv * hd, D),
         "self_attn.v_proj.weight": mk(Hkv * hd, D), "self_attn.o_proj.weight": mk(D, Hq * hd),
         "mlp.gate_proj.weight": mk(I, D), "mlp.up_proj.weight": mk(I, D), "mlp.down_proj.weight": mk(D, I),
         "input_layernorm.weight": 1 + mk(D), "post_attention_layernorm.weight": 1 + mk(D)}
    if bias:
        w.update({"self_attn.q_proj.bias": mk(Hq * hd), "self_attn.k_proj.bias": mk(Hkv * hd), "self_attn.v_proj.bias": mk(Hkv * hd)})
    w = {k: (v.to(DT[dtype]) if v.dim() == 2 else v) for k, v in w.items()}
    mixer_spec = PartSpec("gqa_attention", {"hidden_size": D, "num_heads": Hq, "num_kv_heads": Hkv, "head_dim": hd,
                                            "scale": hd ** -0.5, "window": window, "position": "rope"})
    rope = build(POSITIONS, "position encoding", PartSpec("rope", {"head_dim": hd, "theta": 1e4}))
    rope.prepare(128, torch.device("cuda:0"))
    ctx.positions = {"rope": rope}
    cos, sin = plain_model.rope_tables(hd, 1e4, None, T)
    cfg = dict(Hq=Hq, Hkv=Hkv, hd=hd, eps=1e-5, windows=[window])
    pw = {"model.layers.0." + k: v for k, v in w.items()}
    # --- the mixer alone
    mixer = build(MIXERS, "mixer", mixer_spec)
    mixer.bind({k[len("self_attn."):]: v.cuda() for k, v in w.items() if k.startswith("self_attn.")}, ops)
    h = torch.randn(T, D, generator=g).to(DT[dtype])
    ref = plain_model.attention_layer(h.float(), pw, "model.layers.0.", cfg, cos, sin, window, DT[dtype])
    got = []
    for req, (lo, hi) in (("a", (0, cut)), ("a", (cut, T))):
        cache.ensure(req, hi)
        meta.fill(cache, [Portion(req, [0] * (hi - lo), [])], [lo], ops=ops, needs=("attention",))
        lc = LayerCache(*cache.groups[0].view(0), group=0, page_size=8, write=True)
        got.append(mixer.forward(ctx, h[lo:hi].cuda(), lc).cpu().clone())
        cache.commit(req, hi)
    got = torch.cat(got)
    assert float((got - ref).abs().max()) <= tol(dtype, ref, 3.0), float((got - ref).abs().max())
    # --- the block (norms + mixer + feed-forward), second cache slot, one portion
    block = BLOCKS["pre_norm"](build(MIXERS, "mixer", mixer_spec),
                               build(FEED_FORWARDS, "feed-forward", PartSpec("swiglu", {"hidden_size": D, "intermediate_size": I})),
                               lambda: build(NORMS, "norm", PartSpec("rmsnorm", {"size": D, "eps": 1e-5})))
    assert set(block.tensors()) >= set(w)
    block.bind({k: v.cuda() for k, v in w.items()}, ops)
    x = torch.randn(T, D, generator=g)
    cache.ensure("b", T)
    meta.fill(cache, [Portion("b", [0] * T, [])], [0], ops=ops, needs=("attention",))
    lc = LayerCache(*cache.groups[0].view(1), group=0, page_size=8, write=True)
    xc = x.clone().cuda()
    x_out, delta = block.forward(ctx, xc, None, lc)
    full = plain_model.layer(x, pw, 0, cfg, cos, sin, DT[dtype])
    res = (x_out + delta).cpu()
    assert float((res - full).abs().max()) <= tol(dtype, full, 3.0), float((res - full).abs().max())
    ops.check_errors()
