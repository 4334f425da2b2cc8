"""A plain PyTorch kernel table with the meanings of `fusezap_core_b200.kernels.interface.Ops`.

Two uses: (1) the plain reference of every CUDA kernel in the `-m gpu` kernel tests (called with CPU copies of the
same inputs); (2) the `-m "not gpu"` tests hand it to the engine in place of the CUDA table, so the host-side logic
(step metadata, block tables, page reuse, the scheduler) is exercised on the CPU. It is never on the product path.
"""
from __future__ import annotations
import numpy as np
import torch

import plain_model


class PlainOps:
    def __init__(self, dtype: torch.dtype = torch.float32):
        self.dtype = dtype
        self.launches = 0

    def check_attention(self, num_heads, num_kv_heads, head_dim) -> None:
        if num_heads % num_kv_heads or head_dim % 2:
            raise ValueError("bad attention sizes")

    def embed(self, table, tokens, x, src=None, prev_ids=None, scale=1.0) -> None:
        t = tokens.long()
        if src is not None:
            t = torch.where(src >= 0, prev_ids.long()[src.long().clamp(min=0)], t)
        if ((t < 0) | (t >= table.shape[0])).any():
            raise ValueError("token id outside the embedding table")
        x.copy_(table[t].float() * torch.tensor(scale, dtype=torch.float32))

    def add_rmsnorm(self, x, delta, weight, eps, h, rows=None) -> None:
        if rows is None:
            if delta is not None:
                x.add_(delta)
            src = x
        else:
            r = rows.long().clamp(min=0)
            src = x[r] + (delta[r] if delta is not None else 0)
        y = src * torch.rsqrt((src * src).mean(-1, keepdim=True) + eps)
        y = weight.float() * y
        if rows is not None:
            y = torch.where((rows < 0)[:, None], torch.zeros_like(y), y)
        h.copy_(y.to(h.dtype))

    def linear(self, a, w, bias, out) -> None:
        y = a.float() @ w.float().T
        if bias is not None:
            y = y + bias.float()
        out.copy_(y.to(out.dtype))

    def rope_kv_write(self, qkv, cos, sin, meta, cache, q_out, num_heads, num_kv_heads, head_dim) -> None:
        n, Hq, Hkv, hd = qkv.shape[0], num_heads, num_kv_heads, head_dim
        pos, row = meta.pos.long(), meta.seq_row.long()
        x = qkv.view(n, Hq + 2 * Hkv, hd)
        c, s = cos[pos][:, None, :], sin[pos][:, None, :]
        qk = x[:, :Hq + Hkv]
        x1, x2 = qk[..., :hd // 2], qk[..., hd // 2:]
        rot = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)
        live = row >= 0
        q = torch.where(live[:, None, None], rot[:, :Hq], torch.zeros(()))
        q_out.copy_(q.reshape(n, Hq * hd).to(q_out.dtype))
        if not cache.write:
            return
        table = meta.table(cache.group)
        bs = cache.page_size
        for i in range(n):
            if row[i] < 0:
                continue
            page = int(table[row[i], pos[i] // bs])
            assert page >= 0, f"row {i} at position {int(pos[i])} has no page"
            cache.keys[page, :, pos[i] % bs, :] = rot[i, Hq:].to(cache.keys.dtype)
            cache.values[page, :, pos[i] % bs, :] = x[i, Hq + Hkv:].to(cache.values.dtype)

    def paged_attention(self, q, cache, meta, out, num_heads, num_kv_heads, head_dim, scale, window) -> None:
        n, Hq, Hkv, hd = q.shape[0], num_heads, num_kv_heads, head_dim
        G = Hq // Hkv
        pos, row = meta.pos.long(), meta.seq_row.long()
        table = meta.table(cache.group)
        bs = cache.page_size
        o = torch.zeros(n, Hq, hd)
        for i in range(n):
            if row[i] < 0:
                continue
            p = int(pos[i])
            lo = max(0, p - window + 1) if window else 0
            js = torch.arange(lo, p + 1)
            pages = table[row[i], js // bs].long()
            assert (pages >= 0).all(), f"row {i}: a visible key's page was given back"
            K = cache.keys[pages, :, js % bs, :].float()       # (keys, Hkv, hd)
            V = cache.values[pages, :, js % bs, :].float()
            qi = q[i].float().view(Hq, hd)
            for h in range(Hq):
                s = (K[:, h // G, :] @ qi[h]) * scale
                o[i, h] = torch.softmax(s, 0) @ V[:, h // G, :]
        out.copy_(o.reshape(n, Hq * hd).to(out.dtype))

    def pack_gate_up(self, gate, up, gate_bias=None, up_bias=None):
        return None

    def swiglu(self, gate_up, out) -> None:
        I = out.shape[1]
        g, u = gate_up[:, :I].float(), gate_up[:, I:].float()
        out.copy_((g / (1 + torch.exp(-g)) * u).to(out.dtype))

    def argmax(self, logits, out) -> None:
        a = logits.detach().cpu().numpy()
        out.copy_(torch.from_numpy(np.argmax(a, axis=-1).astype(np.int32)))

    def sample(self, logits, temperature, uniform, out) -> None:
        a = logits.detach().cpu().numpy()
        res = np.zeros(a.shape[0], np.int32)
        for r in range(a.shape[0]):
            t = float(temperature[r])
            if t <= 0:
                res[r] = int(np.argmax(a[r]))
                continue
            x = a[r].astype(np.float64) / t
            e = np.exp(x - x.max())
            c = np.cumsum(e)
            res[r] = int(np.searchsorted(c, float(uniform[r]) * c[-1], side="right").clip(0, len(c) - 1))
        out.copy_(torch.from_numpy(res))

    def sample_filtered(self, logits, temperature, top_k, top_p, uniform, out) -> None:
        a = logits.detach().cpu().numpy()
        res = np.zeros(a.shape[0], np.int32)
        for r in range(a.shape[0]):
            t, k, p = float(temperature[r]), int(top_k[r]), float(top_p[r])
            if t <= 0 or k == 1:
                res[r] = int(np.argmax(a[r]))
                continue
            x = plain_model.top_p_filter(plain_model.top_k_filter(a[r].astype(np.float64) / t, k), p)
            c = np.cumsum(np.exp(x - x.max()))
            res[r] = int(np.searchsorted(c, float(uniform[r]) * c[-1], side="right").clip(0, len(c) - 1))
        out.copy_(torch.from_numpy(res))

    def errors_to_host(self) -> None:
        pass

    def check_errors(self, copied: bool = False) -> None:
        pass
