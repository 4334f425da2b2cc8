"""The description of a model leaves room for more than the dense decoder uses: norms of different kinds in one layer
(named by the block's params), a scale on the embeddings, a transform of the logits, and models without any attention
layer (which then carry no attention step data). Toy parts defined here fill those places without a change to the
package; the result is compared with a plain restatement. Runs on the CPU with the plain kernel table, and once more
on the GPU with the CUDA kernels."""
import math

import numpy as np
import pytest
import torch

from fusezap_core_b200.cache import CacheManager
from fusezap_core_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from fusezap_core_b200.engine import Portion, StepRunner
from fusezap_core_b200.engine.model import DecoderModel
from fusezap_core_b200.parts import (LOGIT_TRANSFORMS, MIXERS, NORMS, LogitTransform, Mixer, Norm, register_logit_transform,
                                     register_mixer, register_norm)
from fusezap_core_b200.weights import ParamSpec
from plain_ops import PlainOps

D, V, CAP, EPS = 32, 61, 3.0, 1e-5


@pytest.fixture(scope="module", autouse=True)
def toy_parts():
    @register_norm("toy_mean_abs")
    class MeanAbsNorm(Norm):
        """h = w * x / (mean|x| + eps): another kind of norm than RMSNorm, with the same interface."""
        def __init__(self, size: int, eps: float):
            self.size, self.eps = size, eps
        def tensors(self):
            return {"weight": ParamSpec((self.size,), role="vector", init="ones")}
        def bind(self, tensors, ops):
            self.weight = tensors["weight"]
        def forward(self, ctx, x, delta, rows=None, n_rows=None):
            if delta is not None:
                x.add_(delta)
            h = self.weight.float() * x / (x.abs().mean(-1, keepdim=True) + self.eps)
            return h.to(ctx.ops.dtype)

    @register_mixer("toy_shift")
    class Shift(Mixer):
        """A mixer without cache or state: a linear map of the token's own row."""
        def __init__(self, hidden_size: int):
            self.D = hidden_size
        def tensors(self):
            return {"proj.weight": ParamSpec((self.D, self.D))}
        def bind(self, tensors, ops):
            self.w = {"proj": tensors["proj.weight"]}      # kept in a dict: weight_tensors() has to say so
        def weight_tensors(self):
            return list(self.w.values())
        def forward(self, ctx, h, cache):
            out = ctx.ws.get("toy_shift", (h.shape[0], self.D), torch.float32)
            ctx.ops.linear(h, self.w["proj"], None, out)
            return out

    @register_logit_transform("toy_soft_cap")
    class SoftCap(LogitTransform):
        def __init__(self, cap: float):
            self.cap = cap
        def forward(self, ctx, logits):
            logits.copy_(torch.tanh(logits / self.cap) * self.cap)
    yield
    NORMS.pop("toy_mean_abs", None); MIXERS.pop("toy_shift", None); LOGIT_TRANSFORMS.pop("toy_soft_cap", None)


def spec(with_attention: bool) -> ModelSpec:
    rms = PartSpec("rmsnorm", {"size": D, "eps": EPS})
    mean_abs = PartSpec("toy_mean_abs", {"size": D, "eps": EPS})
    ffn = PartSpec("swiglu", {"hidden_size": D, "intermediate_size": 2 * D})
    attn = PartSpec("gqa_attention", {"hidden_size": D, "num_heads": 2, "num_kv_heads": 1, "head_dim": 16, "scale": 0.25,
                                      "window": 0, "position": "rope"})
    # layer 0: two norm kinds in one layer, named by the block's params; no fallback norm on the layer at all
    layers = [LayerSpec("m.0.", PartSpec("pre_norm", {"norms": (mean_abs, rms)}), PartSpec("toy_shift", {"hidden_size": D}), ffn)]
    if with_attention:
        layers.append(LayerSpec("m.1.", PartSpec("pre_norm"), attn, ffn, rms))
    return ModelSpec(architecture="toy_slots", hidden_size=D, vocab_size=V, embed_name="m.embed.weight", lm_head_name=None,
                     tie_embeddings=True, final_norm=rms, final_norm_name="m.norm.weight", layers=tuple(layers),
                     schedule=tuple(ScheduleEntry(i, i) for i in range(len(layers))),
                     positions={"rope": PartSpec("rope", {"head_dim": 16, "theta": 100.0})}, max_position=64,
                     embed_scale=math.sqrt(D), logit_transform=PartSpec("toy_soft_cap", {"cap": CAP}))


def weights(model: DecoderModel, seed: int) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, p in model.expected_tensors().items():
        if p.ignore or p.group is not None:
            continue
        out[name] = 1 + 0.1 * torch.randn(p.shape, generator=g) if p.init == "ones" else torch.randn(p.shape, generator=g) * 0.3
    return out


def plain(w, ids, with_attention: bool) -> torch.Tensor:
    rms = lambda x, wt: wt * x * torch.rsqrt((x * x).mean(-1, keepdim=True) + EPS)
    swiglu = lambda h, p: (torch.nn.functional.silu(h @ w[p + "mlp.gate_proj.weight"].T) * (h @ w[p + "mlp.up_proj.weight"].T)) @ w[p + "mlp.down_proj.weight"].T
    x = w["m.embed.weight"][torch.tensor(ids)] * torch.tensor(math.sqrt(D), dtype=torch.float32)
    T = len(ids)
    h = w["m.0.input_layernorm.weight"] * x / (x.abs().mean(-1, keepdim=True) + EPS)
    x = x + h @ w["m.0.self_attn.proj.weight"].T
    x = x + swiglu(rms(x, w["m.0.post_attention_layernorm.weight"]), "m.0.")
    if with_attention:
        h = rms(x, w["m.1.input_layernorm.weight"])
        inv = 1.0 / (100.0 ** (torch.arange(0, 16, 2).float() / 16))
        ang = torch.arange(T).float()[:, None] * inv[None]
        def rot(t):
            a, b = t[..., :8], t[..., 8:]
            return torch.cat([a * ang.cos()[:, None] - b * ang.sin()[:, None], b * ang.cos()[:, None] + a * ang.sin()[:, None]], -1)
        q = rot((h @ w["m.1.self_attn.q_proj.weight"].T).view(T, 2, 16))
        k = rot((h @ w["m.1.self_attn.k_proj.weight"].T).view(T, 1, 16))
        v = (h @ w["m.1.self_attn.v_proj.weight"].T).view(T, 1, 16)
        o = torch.zeros(T, 2, 16)
        for hh in range(2):
            sc = (q[:, hh] @ k[:, 0].T) * 0.25
            sc = sc.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
            o[:, hh] = torch.softmax(sc, -1) @ v[:, 0]
        x = x + o.reshape(T, 32) @ w["m.1.self_attn.o_proj.weight"].T
        x = x + swiglu(rms(x, w["m.1.post_attention_layernorm.weight"]), "m.1.")
    lg = rms(x, w["m.norm.weight"]) @ w["m.embed.weight"].T
    return torch.tanh(lg / CAP) * CAP


def build(with_attention: bool, ops, device):
    model = DecoderModel(spec(with_attention))
    w = weights(model, seed=5)
    model.ops = ops
    model.bind({k: v.to(device) for k, v in w.items()}, ops, "float32", torch.device(device), 64)
    return model, w


def check(model, w, with_attention, device):
    cache = CacheManager(model.cache_needs(), model.state_needs(), 8, 16, 2, 64, torch.float32, device)
    run = StepRunner(model, cache, max_rows=64)
    ids = np.random.default_rng(0).integers(0, V, 37).tolist()
    got = torch.cat([run.run([Portion("a", ids[:20], list(range(20)))]).cpu().clone(),
                     run.run([Portion("a", ids[20:22], [0, 1])]).cpu().clone(),
                     run.run([Portion("a", ids[22:], list(range(15)))]).cpu().clone()])
    ref = plain(w, ids, with_attention)
    assert float(ref.abs().max()) <= CAP and float(ref.abs().max()) > 0.5 * CAP, "the cap is at work"
    np.testing.assert_allclose(got.numpy(), ref.numpy(), rtol=1e-4, atol=2e-5)
    return run


@pytest.mark.parametrize("with_attention", [False, True])
def test_slots_on_the_cpu(with_attention):
    model, w = build(with_attention, PlainOps(), "cpu")
    run = check(model, w, with_attention, "cpu")
    assert run.needs == (("attention",) if with_attention else ())
    shift = model.layers[0].mixer
    n_shift = sum(t.numel() * 4 for t in shift.weight_tensors())
    assert n_shift == D * D * 4 and model.weight_bytes() >= n_shift + V * D * 4, "a part that keeps tensors in a dict is counted"
    kinds = {type(p).__name__ for p in model.parts()}
    assert {"MeanAbsNorm", "RMSNorm", "Shift", "SoftCap", "SwiGLU", "PreNormBlock"} <= kinds


def test_a_layer_without_a_norm_for_its_block_is_refused():
    s = spec(False)
    import dataclasses
    bad = dataclasses.replace(s, layers=(dataclasses.replace(s.layers[0], block=PartSpec("pre_norm")),))
    with pytest.raises(ValueError, match="asks for a norm"):
        DecoderModel(bad)


@pytest.mark.gpu
@pytest.mark.parametrize("with_attention", [False, True])
def test_slots_on_the_gpu(with_attention):
    from fusezap_core_b200.kernels import cuda_ops
    model, w = build(with_attention, cuda_ops("float32", "cuda:0"), "cuda:0")
    run = check(model, w, with_attention, "cuda:0")
    model.ops.check_errors()
    if with_attention:
        assert run.meta.extra_ints > 0 and run.meta.plan is not None and run.meta.plan.n_tiles == 1
    else:
        assert run.meta.extra_ints == 0 and run.meta.plan is None, "a model without attention carries no tile list"
