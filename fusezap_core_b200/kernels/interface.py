"""The kernel table: every device operation a part may ask for, with its exact meaning.

The product has one implementation, `CudaOps` (hand-written sm_100a kernels; it refuses tensors that are not on a
GPU and raises if its library cannot be built or loaded). The interface exists so that parts depend on meanings, not on
launch details, and so that a test can hand the same engine a plain PyTorch table to check the host-side logic without
a GPU.

Conventions. N: token rows of the step. T: the activation dtype (`ops.dtype`: float32 or bfloat16). The residual stream
and every sublayer output are float32. Rows whose `meta.seq_row` is negative are padding: kernels write zeros for them
and store nothing in the cache. All sums over a row, a head or a key range are in 32-bit and their order depends only
on the row's own data, never on the other rows of the step.
"""
from __future__ import annotations
from typing import Any

import torch


class Ops:
    dtype: torch.dtype

    def step_extra_ints(self, needs: tuple, max_rows: int, max_segments: int) -> int:
        """How many int32 of the step's metadata block this table wants for itself, given the kinds of step data the
        model's mixers need (`Mixer.step_needs()`), for steps of at most max_rows rows of at most max_segments requests."""
        return 0

    def plan_step(self, meta: Any, needs: tuple) -> None:
        """Called once per step, after the metadata is packed on the host and before its copy to the device: the table
        may fill `meta.extra_host` (its int32 in the block) and keep launch sizes in `meta.plan`."""

    def step_signature(self, meta: Any) -> tuple:
        """What, beside the numbers of rows and wanted rows, fixes the kernel launches of the step just planned; two
        steps with equal signatures may replay one captured graph."""
        return ()

    def check_attention(self, num_heads: int, num_kv_heads: int, head_dim: int) -> None:
        """Raise ValueError if the attention kernels cannot take these sizes (nothing is ever computed wrongly)."""
        raise NotImplementedError

    def embed(self, table: torch.Tensor, tokens: torch.Tensor, x: torch.Tensor, src: torch.Tensor | None = None,
              prev_ids: torch.Tensor | None = None, scale: float = 1.0) -> None:
        """x[n, :] = float32(table[tokens[n], :]) * scale. tokens: int32 (N,). A token outside the table is an error.
        With src (int32 (N,)) and prev_ids (int32): a row with src[n] >= 0 uses token prev_ids[src[n]] instead."""
        raise NotImplementedError

    def add_rmsnorm(self, x: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float,
                    h: torch.Tensor, rows: torch.Tensor | None = None) -> None:
        """rows None: x += delta (if given), in place; h[n] = T(weight * x[n] / sqrt(mean(x[n]^2) + eps)).
        rows (int32 (R,), -1 = none): h[r] is computed from x[rows[r]] + delta[rows[r]]; x is not written."""
        raise NotImplementedError

    def linear(self, a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor) -> None:
        """out[m, n] = sum_k a[m, k] * w[n, k] (+ bias[n]); a: (M, K) T, w: (N, K) T, bias float32, out float32 or T;
        accumulation in float32, one rounding into out."""
        raise NotImplementedError

    def pack_gate_up(self, gate: torch.Tensor, up: torch.Tensor, gate_bias: torch.Tensor | None = None,
                     up_bias: torch.Tensor | None = None):
        """Prepares the gate and up matrices ((I, K) each) for `linear_swiglu` in whatever layout the kernels want, or
        returns None if this table has no fused kernel for these sizes (the part then runs `linear` + `swiglu`)."""
        return None

    def linear_swiglu(self, a: torch.Tensor, packed: Any, out: torch.Tensor) -> None:
        """out[m, i] = T(silu(a[m] . gate[i] + gate_bias[i]) * (a[m] . up[i] + up_bias[i])); `packed` from `pack_gate_up`.
        The products are accumulated in float32 and are not rounded before the activation."""
        raise NotImplementedError

    def rope_kv_write(self, qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, meta: Any, cache: Any,
                      q_out: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int) -> None:
        """qkv: (N, (Hq + 2 Hkv) * hd) float32, heads [q | k | v]. Rotates q and k heads by the row's position
        (pairs j, j + hd/2, angles from the float32 tables cos/sin (max_len, hd/2)); writes q to q_out (N, Hq*hd) T
        and, if cache.write, k and v to the row's page slot of cache.keys / cache.values."""
        raise NotImplementedError

    def linear_rope_kv_write(self, a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, cos: torch.Tensor,
                             sin: torch.Tensor, meta: Any, cache: Any, q_out: torch.Tensor, num_heads: int,
                             num_kv_heads: int, head_dim: int) -> bool:
        """`linear` (a . w^T + bias, w rows = [q heads | k heads | v heads]) followed by `rope_kv_write` on its float32
        result, as one operation that never writes that result out. Returns False, having done nothing, if this table
        has no such kernel for these sizes; the caller then runs the two operations."""
        return False

    def paged_attention(self, q: torch.Tensor, cache: Any, meta: Any, out: torch.Tensor, num_heads: int,
                        num_kv_heads: int, head_dim: int, scale: float, window: int) -> None:
        """out[n, h] = softmax_j((q[n, h] . K[j]) * scale) V[j] over the keys j of the row's own request with
        max(0, p - window + 1) <= j <= p (window 0: 0 <= j <= p), p = meta.pos[n]; kv head h // (Hq / Hkv)."""
        raise NotImplementedError

    def swiglu(self, gate_up: torch.Tensor, out: torch.Tensor) -> None:
        """gate_up: (N, 2 I) T = [gate | up]; out[n, i] = T(silu(gate[n, i]) * up[n, i]), silu in float32."""
        raise NotImplementedError

    def linear_argmax(self, a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor) -> bool:
        """out[m] = argmax_n (a[m] . w[n] + bias[n]) (the order of `argmax` below) without writing the products out.
        Optional: returns False, having done nothing, if this table has no such kernel for these sizes."""
        return False

    def argmax(self, logits: torch.Tensor, out: torch.Tensor) -> None:
        """out[r] = first index of the row's maximum (a NaN counts as the maximum, the first one wins); int32."""
        raise NotImplementedError

    def sample(self, logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor, out: torch.Tensor) -> None:
        """out[r] = the token at which the running sum of softmax(logits[r] / temperature[r]) (float64, in index
        order) first exceeds uniform[r] * total; temperature[r] <= 0 means argmax. uniform: float64 in [0, 1)."""
        raise NotImplementedError

    def sample_filtered(self, logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
                        uniform: torch.Tensor, out: torch.Tensor) -> None:
        """`sample` after the reference's filters on logits[r] / temperature[r] (fusezap/serve/sampling.py:25-45):
        top_k[r] (int32; <= 0 or >= V: off, 1: argmax) keeps what is not below the k-th largest value, ties included;
        top_p[r] (float32; >= 1: off) then keeps, in falling order of value and rising index among equals, every token
        before which less than top_p[r] of the probability lies."""
        raise NotImplementedError
