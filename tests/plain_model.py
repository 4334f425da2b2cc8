"""A plain, slow implementation of the dense Llama / Qwen2.5 decoder: whole sequences, no cache, one function per part.

It shares no code with the package: it reads config.json keys and checkpoint tensor names itself and computes with
plain PyTorch on the CPU in float32. Every function cites the reference lines (paths inside fusezap/fusezap-core) whose
formula it restates. `tests/golden/` holds logits of the reference's own model code (run on its numpy device) for the
tiny configurations; `test_plain_model.py` checks this file against them.

`act_dtype=torch.bfloat16` rounds at the places where the engine's bfloat16 path stores an activation in bfloat16 (norm
output, q, cached k and v, attention output, gate/up output, the SwiGLU product); everything else stays float32, as in
the engine (residual stream, scores, softmax, sums, logits).
"""
from __future__ import annotations
import math

import numpy as np
import torch


def _rt(x: torch.Tensor, dt: torch.dtype) -> torch.Tensor:
    """Round to the activation dtype and come back to float32."""
    return x if dt == torch.float32 else x.to(dt).to(torch.float32)


# ---------------------------------------------------------------- configuration (fusezap/serve/models/llama.py:78-100)
def read_config(c: dict) -> dict:
    heads = c["num_attention_heads"]
    rp = c.get("rope_parameters") or {}
    theta = c.get("rope_theta") or rp.get("rope_theta") or 10000.0                                   # llama.py:87
    scaling = c.get("rope_scaling") or ({k: v for k, v in rp.items() if k != "rope_theta"}
                                        if rp.get("rope_type", "default") != "default" else None)   # llama.py:88
    n_layers = c["num_hidden_layers"]
    windows = [0] * n_layers
    if c.get("use_sliding_window", False) and c.get("sliding_window"):                               # llama.py:94, 99
        types = c.get("layer_types") or ["sliding_attention"] * n_layers                            # swa.py:24-30
        windows = [int(c["sliding_window"]) if t == "sliding_attention" else 0 for t in types]
    return dict(D=c["hidden_size"], I=c["intermediate_size"], L=n_layers, Hq=heads,
                Hkv=c.get("num_key_value_heads") or heads, hd=c.get("head_dim") or c["hidden_size"] // heads,
                V=c["vocab_size"], eps=c.get("rms_norm_eps", 1e-6), theta=float(theta), scaling=scaling,
                tie=bool(c.get("tie_word_embeddings", False)), windows=windows)


# ---------------------------------------------------------------- position encoding
def rope_inv_freq(hd: int, theta: float, scaling: dict | None) -> np.ndarray:
    """fusezap/serve/models/llama.py:102-120."""
    inv = (1.0 / (np.float32(theta) ** (np.arange(0, hd, 2, dtype=np.int64).astype(np.float32) / np.float32(hd)))).astype(np.float32)
    rs = scaling or {}
    kind = rs.get("rope_type", rs.get("type"))
    if kind == "linear":
        inv = (inv / np.float32(rs["factor"])).astype(np.float32)
    elif kind == "llama3":
        f, lo, hi = rs["factor"], rs.get("low_freq_factor", 1.0), rs.get("high_freq_factor", 4.0)
        old = rs["original_max_position_embeddings"]
        wl = 2 * math.pi / inv
        smooth = (old / wl - lo) / (hi - lo)
        out = np.where(wl > old / lo, inv / f, inv)
        mid = (wl <= old / lo) & (wl >= old / hi)
        inv = np.where(mid, (1 - smooth) * out / f + smooth * out, out).astype(np.float32)
    elif kind not in (None, "default"):
        raise NotImplementedError(kind)
    return inv


def rope_tables(hd: int, theta: float, scaling: dict | None, n: int) -> tuple[torch.Tensor, torch.Tensor]:
    """fusezap/serve/models/llama.py:122-130: (n, hd/2) cos and sin of float32(position) * inv_freq, float32."""
    fr = np.arange(n, dtype=np.float32)[:, None] * rope_inv_freq(hd, theta, scaling)[None, :]
    return torch.from_numpy(np.cos(fr).astype(np.float32)), torch.from_numpy(np.sin(fr).astype(np.float32))


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """fusezap/serve/models/llama.py:524-527. x: (T, H, hd); cos, sin: (T, hd/2)."""
    h = x.shape[-1] // 2
    x1, x2 = x[..., :h], x[..., h:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c + (-x2) * s, x2 * c + x1 * s], dim=-1)


# ---------------------------------------------------------------- norm
def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """fusezap/serve/models/llama.py:500-503: x * rsqrt(mean(x^2) + eps), times the weight."""
    xf = x.float()
    return w.float() * (xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps))


# ---------------------------------------------------------------- mixer
def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: int) -> torch.Tensor:
    """fusezap/serve/models/llama.py:587-594 with the mask of fusezap/serve/models/swa.py:74-77.
    q: (T, Hq, hd); k, v: (T, Hkv, hd); query t sees keys j <= t (and j > t - window if window). -> (T, Hq*hd)."""
    T, Hq, hd = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    qpos = torch.arange(T)[:, None]
    kpos = torch.arange(T)[None, :]
    mask = kpos <= qpos
    if window:
        mask = mask & (kpos > qpos - window)
    out = torch.empty(T, Hq, hd)
    for h in range(Hq):
        s = (q[:, h, :] @ k[:, h // G, :].T) * scale
        s = torch.where(mask, s, torch.tensor(float("-inf")))
        out[:, h, :] = torch.softmax(s, dim=-1) @ v[:, h // G, :]
    return out.reshape(T, Hq * hd)


def attention_layer(h: torch.Tensor, w: dict, p: str, cfg: dict, cos, sin, window: int, dt) -> torch.Tensor:
    """fusezap/serve/models/llama.py:570-600: q/k/v projections (+ bias when the checkpoint has one), rotation of q
    and k, attention, output projection."""
    T = h.shape[0]
    Hq, Hkv, hd = cfg["Hq"], cfg["Hkv"], cfg["hd"]
    def proj(name):
        y = h @ w[p + f"self_attn.{name}.weight"].float().T
        b = w.get(p + f"self_attn.{name}.bias")
        return y + b.float() if b is not None else y
    q = _rt(apply_rope(proj("q_proj").reshape(T, Hq, hd), cos, sin), dt)
    k = _rt(apply_rope(proj("k_proj").reshape(T, Hkv, hd), cos, sin), dt)
    v = _rt(proj("v_proj").reshape(T, Hkv, hd), dt)
    o = _rt(attention(q, k, v, 1.0 / math.sqrt(hd), window), dt)                                    # llama.py:557
    y = o @ w[p + "self_attn.o_proj.weight"].float().T
    b = w.get(p + "self_attn.o_proj.bias")
    return y + b.float() if b is not None else y


# ---------------------------------------------------------------- feed-forward
def silu(g: torch.Tensor) -> torch.Tensor:
    """fusezap/serve/cuda.py:284-303: g * 1 / (1 + exp(-g))."""
    return g / (1.0 + torch.exp(-g))


def swiglu_mlp(h: torch.Tensor, w: dict, p: str, dt) -> torch.Tensor:
    """fusezap/serve/models/llama.py:601-606, 746-752."""
    def lin(name, x):
        y = x @ w[p + f"mlp.{name}.weight"].float().T
        b = w.get(p + f"mlp.{name}.bias")
        return y + b.float() if b is not None else y
    g, u = _rt(lin("gate_proj", h), dt), _rt(lin("up_proj", h), dt)
    return lin("down_proj", _rt(silu(g) * u, dt))


# ---------------------------------------------------------------- block and model
def layer(x: torch.Tensor, w: dict, i: int, cfg: dict, cos, sin, dt, cache_of: dict | None = None) -> torch.Tensor:
    """Pre-norm block (fusezap/serve/models/llama.py:568, 600-606): x += attn(norm1(x)); x += mlp(norm2(x))."""
    p = f"model.layers.{i}."
    h = _rt(rmsnorm(x, w[p + "input_layernorm.weight"], cfg["eps"]), dt)
    x = x + attention_layer(h, w, p, cfg, cos, sin, cfg["windows"][i], dt)
    h = _rt(rmsnorm(x, w[p + "post_attention_layernorm.weight"], cfg["eps"]), dt)
    return x + swiglu_mlp(h, w, p, dt)


def forward(config: dict, weights: dict, ids, act_dtype: torch.dtype = torch.float32,
            schedule: list[int] | None = None) -> torch.Tensor:
    """Logits (T, V) float32 for every position of one whole sequence (fusezap/serve/models/llama.py:539-616 with
    last_only=False). weights: checkpoint names -> tensors; with act_dtype bfloat16 pass bfloat16-rounded weights.
    schedule: layer indices in execution order (default 0..L-1)."""
    cfg = read_config(config)
    ids = torch.as_tensor(list(ids), dtype=torch.long)
    T = ids.shape[0]
    cos, sin = rope_tables(cfg["hd"], cfg["theta"], cfg["scaling"], T)
    x = weights["model.embed_tokens.weight"].float()[ids]                                           # llama.py:528-537
    for i in (schedule if schedule is not None else range(cfg["L"])):
        x = layer(x, weights, i, cfg, cos, sin, act_dtype)
    h = _rt(rmsnorm(x, weights["model.norm.weight"], cfg["eps"]), act_dtype)                        # llama.py:614
    head = weights.get("lm_head.weight")
    if cfg["tie"] or head is None:                                                                  # llama.py:362-367
        head = weights["model.embed_tokens.weight"]
    return h @ head.float().T


# ---------------------------------------------------------------- sampling (fusezap/serve/sampling.py)
def apply_repetition_penalty(logits: np.ndarray, history, penalty: float) -> np.ndarray:
    """sampling.py:17-23: a seen token's logit is divided by the penalty if positive, multiplied if negative."""
    if penalty == 1.0 or len(history) == 0:
        return logits
    out = logits.copy()
    idx = np.unique(np.asarray(history, np.int64))
    v = out[idx]
    out[idx] = np.where(v > 0, v / penalty, v * penalty)
    return out


def top_k_filter(logits: np.ndarray, k: int) -> np.ndarray:
    """sampling.py:25-29: ties at the k-th value are kept."""
    if k <= 0 or k >= logits.shape[-1]:
        return logits
    kth = np.partition(logits, -k)[-k]
    return np.where(logits < kth, -np.inf, logits)


def softmax64(x: np.ndarray) -> np.ndarray:
    """sampling.py:31-34."""
    x = np.asarray(x, np.float64)
    e = np.exp(x - np.max(x))
    return e / e.sum()


def top_p_filter(logits: np.ndarray, p: float) -> np.ndarray:
    """sampling.py:36-45: the smallest set of most likely tokens whose mass reaches p; the top one always stays."""
    if p >= 1.0:
        return logits
    order = np.argsort(-logits, kind="stable")
    probs = softmax64(logits)[order]
    cum = np.cumsum(probs)
    drop_sorted = (cum - probs) >= p
    drop = np.zeros_like(drop_sorted)
    drop[order] = drop_sorted
    return np.where(drop, -np.inf, logits)


def sample(logits: np.ndarray, history, temperature: float, top_k: int, top_p: float, repetition_penalty: float,
           rng: np.random.Generator) -> int:
    """sampling.py:61-73: penalty -> temperature -> top-k -> top-p -> softmax (float64) -> one uniform draw."""
    lg = apply_repetition_penalty(np.asarray(logits, np.float32), history, repetition_penalty)
    if temperature == 0 or top_k == 1:
        return int(np.argmax(lg))
    lg = top_p_filter(top_k_filter(lg.astype(np.float64) / temperature, top_k), top_p)
    p = softmax64(lg)
    return int(np.searchsorted(np.cumsum(p), rng.random() * p.sum(), side="right").clip(0, len(p) - 1))
