"""`CudaOps`: the kernel table of the product, hand-written sm_100a kernels called through their C entry points.

Every method checks devices, dtypes and layouts on the host and passes raw pointers and the current CUDA stream to the
library; nothing here computes. A tensor that is not on a CUDA device, a dtype mix the kernels do not take, or a missing
library raises; there is no CPU or library fallback. Kernels that meet bad data (a token outside the table, a position
without a page) set a bit in a device error word instead of faulting; `check_errors()` reads and clears it.
"""
from __future__ import annotations
import ctypes
from ctypes import c_int, c_void_p, c_float, c_longlong

import torch

from .build import load
from .interface import Ops
from .profile import contexts, ideal_linear_bytes

F32, BF16 = 0, 1
_CODE = {torch.float32: F32, torch.bfloat16: BF16}
_STATUS = {1001: "dtype combination not supported", 1002: "shape not supported", 1003: "misaligned operand",
           1004: "size too large for the kernel", 1005: "driver entry point not found", 1006: "tensor map encode failed"}
_DEVICE_ERRORS = {1: "a token id lies outside the embedding table", 2: "a position has no page in its block table",
                  4: "a position lies outside the position tables", 8: "a bounded wait in a kernel gave up",
                  16: "a selected row lies outside the step"}


LONG_PORTION = 8    # attention: portions of at least this many tokens go to the tile (prefill) kernels
TILE_ROWS = 128     # token rows per tile of those kernels


class KernelError(RuntimeError):
    pass


KEY_TILE = 128            # keys per key tile of the tile kernels
PIECE_MIN_TILES = 8       # a piece of a query tile cut along the keys covers at least this many key tiles
MAX_PIECES = 48           # pieces in a step at most (each has a float32 scratch slot per head)
MAX_CUT_TILES = 16        # query tiles of a step that can be cut


def attention_tiles(portions, n_rows: int, cut_keys: bool = True, heads: int = 32, items_per_entry: int = 16, sms: int = 148):
    """How the attention kernels split a step. `portions`: (row of the block table, rows, first position) per request
    in the step. Returns (entries, cuts, short rows).

    entries: the TILE_ROWS-row query tiles of the portions with at least LONG_PORTION tokens as (block-table row, first
    row within the portion, range), the ones with the most keys first. range -1: the entry covers all keys its rows see.
    A step with few query tiles and many keys behind them (a small portion of a long prompt) would leave most SMs
    without work: where the tiles times `heads` (a block's work is a tile and a head) are fewer than three quarters of
    the SMs and a tile has 2,048 keys and more behind it, or fewer than twice the SMs with 8,192 keys and more, tiles are
    cut along the keys into pieces of equal length, at least PIECE_MIN_TILES key tiles each, range =
    first key tile | key tiles << 16, whose partial results a merge kernel adds up. As many pieces are made as give two
    rounds of items for the SMs (`items_per_entry`: heads, or pairs of heads for the kernel that takes two per block).
    The pieces stand first in the list (their index is their scratch slot) and the pieces of one tile stand together.
    cuts: (first entry, entries) per tile that was cut. short rows: the step's other rows (short portions, single tokens
    and padding), which go to the split-key kernel."""
    tiles, long_rows = [], 0
    for seq_row, n, pos0 in portions:
        if n >= LONG_PORTION:
            long_rows += n
            tiles += [(pos0 + min(r + TILE_ROWS, n), seq_row, r) for r in range(0, n, TILE_ROWS)]
    tiles.sort(key=lambda t: -t[0])
    short = n_rows - long_rows
    key_tiles = [(last - 1) // KEY_TILE + 1 for last, _, _ in tiles]
    total = sum(key_tiles)
    # (measured through the engine at 32 heads and 8 layers: with at least 0.75 items per SM the cuts pay from about
    # 8,192 keys on: a 32,000-token prompt in portions of 768 took 226 ms without them and 198 ms with them, in portions
    # of 1,024 198 and 189 ms; a 7,680-token prompt in portions of 512 38.0 ms without and 38.8 ms with)
    items = len(tiles) * heads
    enough = 2 * PIECE_MIN_TILES if 4 * items < 3 * sms else 8 * PIECE_MIN_TILES
    if not cut_keys or not tiles or items >= 2 * sms or key_tiles[0] < enough or key_tiles[0] >= 1 << 15:
        return [(s, r, -1) for _, s, r in tiles], [], short
    target = min(MAX_PIECES, max(2, (2 * sms) // max(1, items_per_entry)))
    pieces, cuts, whole = [], [], []
    for (_, s, r), kt in zip(tiles, key_tiles):
        n = min(kt // PIECE_MIN_TILES, max(1, round(target * kt / total)))
        if n < 2 or len(pieces) + n > MAX_PIECES or len(cuts) >= MAX_CUT_TILES:
            whole.append((s, r, -1))
            continue
        each = -(-kt // n)
        cuts.append((len(pieces), -(-kt // each)))
        pieces += [(s, r, lo | (min(each, kt - lo) << 16)) for lo in range(0, kt, each)]
    return pieces + whole, cuts, short


class AttentionPlan:
    """What `plan_step` keeps about a step for the attention kernels: the device views of the entry list and of the list
    of tiles cut along the keys, and the counts that size the launches."""
    __slots__ = ("tiles", "n_tiles", "n_short_rows", "cuts", "n_cuts", "n_pieces", "single_tokens")

    def __init__(self, tiles: torch.Tensor | None, n_tiles: int, n_short_rows: int, cuts: torch.Tensor | None = None,
                 n_cuts: int = 0, n_pieces: int = 0, single_tokens: bool = False):
        self.tiles, self.n_tiles, self.n_short_rows = tiles, n_tiles, n_short_rows
        self.cuts, self.n_cuts, self.n_pieces = cuts, n_cuts, n_pieces
        # every portion of the step is one token (a decode step): the kernel for short rows then asks for no portion records
        self.single_tokens = single_tokens


def _p(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


class CudaOps(Ops):
    def __init__(self, dtype: str | torch.dtype, device: str | torch.device = "cuda:0"):
        self.dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}.get(dtype, dtype)
        if self.dtype not in _CODE:
            raise ValueError(f"dtype {dtype!r} is not float32 or bfloat16")
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise KernelError(f"the kernels run on a CUDA device only, not on {self.device}")
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device is available; this engine has no CPU path")
        self.core = load("fzb200_core")
        self.err = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._err_host = torch.zeros(1, dtype=torch.int32, pin_memory=True)
        self.launches = 0
        self._stream_handle = None
        self._scratch_bufs: dict[str, torch.Tensor] = {}
        self._retired: list[torch.Tensor] = []      # outgrown scratch: a captured step may still point at it
        self.tc = None
        if self.dtype == torch.bfloat16:
            self.tc = load("fzb200_tc")      # tcgen05 / TMA kernels
        self.use_tensor_cores = self.tc is not None
        self.prefill_tcgen05 = True        # False: long portions on the mma.sync flash-attention kernel
        self.fuse_swiglu = True            # gate/up product and SwiGLU in one kernel where the sizes allow it
        self.fuse_argmax = True            # lm_head product and argmax in one pass where no logits are asked for
        self.fuse_rope = True              # q/k/v product, rotation and cache write in one kernel (few-token steps)
        self.cut_prefill_keys = True       # few query tiles with many keys behind them are cut along the keys
        self._profile = None               # a StepProfile while the engine profiles its steps
        # the fewest query heads, and the fewest items of a query tile on the prompt kernel, among the attention layers
        # that `check_attention` has seen (the plan of a step is shared by its layers)
        self._attn_heads = self._attn_items = 0
        self._sms = torch.cuda.get_device_properties(self.device).multi_processor_count

    # ---- plumbing
    def begin_step(self) -> None:
        """Called by the step function before it launches anything: the kernels of the step all go to the stream that
        is current now (asked for once; it changes when a graph is captured or a caller switches streams)."""
        self._stream_handle = c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        if self._profile is not None:
            self._profile.begin_step()

    def start_profile(self) -> None:
        """From now on a CUDA event is recorded after every launch (see kernels/profile.py)."""
        from .profile import StepProfile
        self._profile = StepProfile(lambda: torch.cuda.Event(enable_timing=True))

    def profile_report(self) -> dict:
        if self._profile is None:
            raise KernelError("start_profile() was not called")
        self._profile.collect(lambda: torch.cuda.synchronize(self.device))
        return self._profile.report()

    def end_step(self) -> None:
        self._stream_handle = None

    def _stream(self) -> c_void_p:
        if self._stream_handle is not None:
            return self._stream_handle
        return c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def _scratch(self, name: str, numel: int, dtype: torch.dtype, zero: bool = False) -> torch.Tensor:
        """A scratch buffer of at least `numel` elements. It only ever grows, and a buffer that was outgrown is kept
        alive, since a captured step that was recorded with it still writes there."""
        buf = self._scratch_bufs.get(name)
        if buf is None or buf.numel() < numel:
            if buf is not None:
                self._retired.append(buf)
            buf = (torch.zeros if zero else torch.empty)(numel, dtype=dtype, device=self.device)
            self._scratch_bufs[name] = buf
        return buf

    def _check(self, status: int, what: str, ideal_bytes: int = 0) -> None:
        self.launches += 1
        if status != 0:
            why = _STATUS.get(status, f"CUDA error {status}")
            raise KernelError(f"{what}: {why}")
        if self._profile is not None:
            self._profile.note(what, ideal_bytes)

    def _want(self, t: torch.Tensor, name: str, dtypes: tuple, dims: int | None = None) -> None:
        if not t.is_cuda:
            raise KernelError(f"{name} is on {t.device}; the kernels take CUDA tensors only")
        if t.dtype not in dtypes:
            raise KernelError(f"{name} has dtype {t.dtype}, expected one of {dtypes}")
        if not t.is_contiguous():
            raise KernelError(f"{name} is not contiguous")
        if dims is not None and t.dim() != dims:
            raise KernelError(f"{name} has {t.dim()} dimensions, expected {dims}")

    def errors_to_host(self) -> None:
        """Enqueues the copy of the error word to pinned memory on the current stream; after the caller's own
        synchronisation `check_errors(copied=True)` reads it without another round trip."""
        self._err_host.copy_(self.err, non_blocking=True)

    def check_errors(self, copied: bool = False) -> None:
        """Raises if any kernel since the last check flagged bad data. copied=False waits for the device first."""
        word = int(self._err_host[0]) if copied else int(self.err.item())
        if word:
            self.err.zero_()
            raise KernelError("a kernel reported: " + "; ".join(m for b, m in _DEVICE_ERRORS.items() if word & b))

    # ---- per-step planning (the step function calls these; it knows nothing of the kernels' tiling)
    def step_extra_ints(self, needs: tuple, max_rows: int, max_segments: int) -> int:
        """int32 this table wants in the step's metadata block for a model whose mixers need `needs`: three per entry of
        the attention tile list (a query tile per TILE_ROWS rows and one more per portion, plus the pieces of tiles cut
        along the keys), two per tile that is cut."""
        if "attention" not in needs:
            return 0
        return 3 * (max_rows // TILE_ROWS + max_segments + MAX_PIECES) + 2 * MAX_CUT_TILES

    def plan_step(self, meta, needs: tuple) -> None:
        """Called when a step has been packed on the host, before its one copy to the device: writes the attention
        kernels' tile list into the block's extra part and keeps the launch sizes in `meta.plan`."""
        if "attention" not in needs:
            meta.plan = None
            return
        # tiles are cut along the keys only for the kernel that can leave partial results (tcgen05, pages TMA can box)
        page = getattr(meta, "page_size", 0)
        can_cut = self.cut_prefill_keys and self.use_tensor_cores and self.prefill_tcgen05 and \
            (page == 8 or (page > 0 and page % 16 == 0))
        entries, cuts, short = attention_tiles(((sg.seq_row, sg.n, sg.pos0) for sg in meta.segments), meta.n_rows, can_cut,
                                               self._attn_heads or 32, self._attn_items or 16, self._sms)
        n_list = (meta.extra_host.size - 2 * MAX_CUT_TILES) // 3
        host = meta.extra_host[:3 * n_list].reshape(-1, 3)
        host[len(entries):] = -1
        if entries:
            host[:len(entries)] = entries
        host_cuts = meta.extra_host[3 * n_list:].reshape(-1, 2)
        host_cuts[len(cuts):] = 0
        if cuts:
            host_cuts[:len(cuts)] = cuts
        meta.plan = AttentionPlan(meta.extra[:3 * n_list].view(-1, 3), len(entries), short, meta.extra[3 * n_list:].view(-1, 2),
                                  len(cuts), sum(c for _, c in cuts), single_tokens=all(sg.n == 1 for sg in meta.segments))

    def step_signature(self, meta) -> tuple:
        """What, beside the row counts, fixes the kernel launches of a step (two steps that agree in it launch alike)."""
        plan = meta.plan
        return (plan.n_tiles, plan.n_short_rows > 0, plan.n_cuts, plan.single_tokens) if plan is not None else ()

    def check_attention(self, num_heads: int, num_kv_heads: int, head_dim: int) -> None:
        if head_dim % 16:
            raise ValueError(f"head_dim {head_dim} is not a multiple of 16; the attention kernels refuse it")
        if self.core.fz_attn_simt_check(c_int(num_heads), c_int(num_kv_heads), c_int(head_dim)) != 0:
            raise ValueError(f"attention sizes not supported: {num_heads} heads, {num_kv_heads} kv heads, head_dim "
                             f"{head_dim} (need heads % kv_heads == 0 and head_dim <= 512)")
        # (the prompt kernel takes two heads of a kv head per block at head size 128, else one)
        items = num_kv_heads * ((num_heads // num_kv_heads + 1) // 2) if head_dim == 128 else num_heads
        self._attn_heads = min(self._attn_heads or num_heads, num_heads)
        self._attn_items = min(self._attn_items or items, items)

    # ---- kernels
    def embed(self, table, tokens, x, src=None, prev_ids=None, scale: float = 1.0) -> None:
        self._want(table, "embedding table", (torch.float32, torch.bfloat16), 2)
        self._want(tokens, "tokens", (torch.int32,), 1)
        self._want(x, "x", (torch.float32,), 2)
        n, d = x.shape
        if tokens.shape[0] != n or table.shape[1] != d:
            raise KernelError(f"embed: tokens {tuple(tokens.shape)}, table {tuple(table.shape)}, x {tuple(x.shape)}")
        if src is not None:
            self._want(src, "src", (torch.int32,), 1)
            self._want(prev_ids, "prev_ids", (torch.int32,), 1)
        self._check(self.core.fz_embed(_p(table), c_int(_CODE[table.dtype]), _p(tokens), _p(src),
                                       _p(prev_ids if src is not None else None), _p(x), c_int(n), c_int(d),
                                       c_int(table.shape[0]), c_float(scale), _p(self.err), self._stream()), "embed",
                    n * d * (table.element_size() + 4))

    def add_rmsnorm(self, x, delta, weight, eps, h, rows=None) -> None:
        self._want(x, "x", (torch.float32,), 2)
        self._want(weight, "norm weight", (torch.float32, torch.bfloat16), 1)
        self._want(h, "h", (torch.float32, torch.bfloat16), 2)
        if delta is not None:
            self._want(delta, "delta", (torch.float32,), 2)
            if delta.shape != x.shape:
                raise KernelError(f"add_rmsnorm: delta {tuple(delta.shape)} vs x {tuple(x.shape)}")
        n_src, d = x.shape
        n_out = n_src
        if rows is not None:
            self._want(rows, "rows", (torch.int32,), 1)
            n_out = rows.shape[0]
        if h.shape != (n_out, d) or weight.shape[0] != d:
            raise KernelError(f"add_rmsnorm: h {tuple(h.shape)}, expected {(n_out, d)}; weight {tuple(weight.shape)}")
        self._check(self.core.fz_add_rmsnorm(_p(x), _p(delta), _p(weight), c_int(_CODE[weight.dtype]), _p(h),
                                             c_int(_CODE[h.dtype]), _p(rows), c_int(n_out), c_int(n_src), c_int(d),
                                             c_float(eps), _p(self.err), self._stream()), "add_rmsnorm",
                    n_out * d * (4 + (8 if delta is not None and rows is None else 4 if delta is not None else 0) + h.element_size()))

    def linear(self, a, w, bias, out) -> None:
        self._want(a, "linear input", (self.dtype,), 2)
        self._want(w, "linear weight", (self.dtype,), 2)
        self._want(out, "linear output", (torch.float32, self.dtype), 2)
        if bias is not None:
            self._want(bias, "linear bias", (torch.float32,), 1)
        m, k = a.shape
        n = w.shape[0]
        if w.shape[1] != k or out.shape != (m, n) or (bias is not None and bias.shape[0] != n):
            raise KernelError(f"linear: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
        self._gemm(a, w, bias, out, m, n, k)

    def _gemm(self, a, w, bias, out, m, n, k) -> None:
        if self.use_tensor_cores and self.tc.fz_gemm_tc_check(_p(a), _p(w), c_int(m), c_int(n), c_int(k)) == 0:
            self._check(self.tc.fz_gemm_tc(
                _p(a), _p(w), _p(bias), _p(out), c_int(_CODE[out.dtype]), c_int(m), c_int(n), c_int(k),
                _p(self.err), self._stream()), "linear (tensor cores)",
                ideal_linear_bytes(m, n, k, 2, 2, out.element_size()))
            return
        self._check(self.core.fz_gemm_simt(_p(a), _p(w), _p(bias), _p(out), c_int(_CODE[a.dtype]),
                                           c_int(_CODE[out.dtype]), c_int(m), c_int(n), c_int(k), self._stream()),
                    "linear", ideal_linear_bytes(m, n, k, a.element_size(), w.element_size(), out.element_size()))

    def pack_gate_up(self, gate, up, gate_bias=None, up_bias=None):
        """Rows in blocks of 128 = [64 gate rows | 64 up rows] of the same 64 features, so that one 128-row tile of the
        tensor-core product holds both halves of its outputs. None when the fused kernel does not apply."""
        i, k = gate.shape
        if not self.use_tensor_cores or not self.fuse_swiglu or gate.dtype != torch.bfloat16 or i % 64 or k % 8:
            return None
        w = torch.stack([gate.view(i // 64, 64, k), up.view(i // 64, 64, k)], 1).reshape(2 * i, k).contiguous()
        b = None
        if gate_bias is not None:
            b = torch.stack([gate_bias.float().view(i // 64, 64), up_bias.float().view(i // 64, 64)], 1).reshape(2 * i).contiguous()
        return (w, b, i)

    def linear_swiglu(self, a, packed, out) -> None:
        w, b, i = packed
        self._want(a, "linear input", (torch.bfloat16,), 2)
        self._want(out, "swiglu output", (torch.bfloat16,), 2)
        m, k = a.shape
        if w.shape != (2 * i, k) or out.shape != (m, i):
            raise KernelError(f"linear_swiglu: a {tuple(a.shape)}, packed {tuple(w.shape)}, out {tuple(out.shape)}")
        self._check(self.tc.fz_gemm_tc_swiglu(_p(a), _p(w), _p(b), _p(out), c_int(m), c_int(i), c_int(k), _p(self.err),
                                              self._stream()), "linear_swiglu (tensor cores)",
                    ideal_linear_bytes(m, 2 * i, k, 2, 2, 1))

    def _pool(self, cache, hkv: int, hd: int):
        k, v = cache.keys, cache.values
        for t, name in ((k, "key pool"), (v, "value pool")):
            if not t.is_cuda or t.dtype != self.dtype:
                raise KernelError(f"{name}: device {t.device}, dtype {t.dtype}; expected CUDA {self.dtype}")
            if t.dim() != 4 or t.shape[1] != hkv or t.shape[3] != hd or t.shape[2] != cache.page_size:
                raise KernelError(f"{name} has shape {tuple(t.shape)}, expected (pages, {hkv}, {cache.page_size}, {hd})")
            if t.stride(3) != 1 or t.stride(2) != hd or t.stride(1) != cache.page_size * hd:
                raise KernelError(f"{name} has strides {t.stride()}: a page's heads must be contiguous")
        if k.stride(0) != v.stride(0):
            raise KernelError("key and value pools have different page strides")
        return k, v, k.stride(0)

    def rope_kv_write(self, qkv, cos, sin, meta, cache, q_out, num_heads, num_kv_heads, head_dim) -> None:
        self._want(qkv, "qkv", (torch.float32,), 2)
        self._want(cos, "cos table", (torch.float32,), 2)
        self._want(sin, "sin table", (torch.float32,), 2)
        self._want(q_out, "q", (self.dtype,), 2)
        n = qkv.shape[0]
        if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim or q_out.shape != (n, num_heads * head_dim) \
                or cos.shape[1] != head_dim // 2 or sin.shape != cos.shape:
            raise KernelError(f"rope_kv_write: qkv {tuple(qkv.shape)}, q {tuple(q_out.shape)}, cos {tuple(cos.shape)}")
        k, v, page_stride = self._pool(cache, num_kv_heads, head_dim)
        table = meta.table(cache.group)
        self._check(self.core.fz_rope_kv_write(
            _p(qkv), _p(cos), _p(sin), _p(meta.pos), _p(meta.seq_row), _p(table), c_int(table.shape[1]), _p(k), _p(v),
            c_longlong(page_stride), c_int(cache.page_size), c_int(1 if cache.write else 0), _p(q_out),
            c_int(_CODE[self.dtype]), c_int(n), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim),
            c_int(cos.shape[0]), _p(self.err), self._stream()), "rope_kv_write")

    def linear_rope_kv_write(self, a, w, bias, cos, sin, meta, cache, q_out, num_heads, num_kv_heads, head_dim) -> bool:
        m, k = a.shape
        if not (self.use_tensor_cores and self.fuse_rope and self.dtype == torch.bfloat16) or \
                self.tc.fz_gemm_tc_qkv_rope_check(c_int(m), c_int(head_dim)) != 0 or \
                self.tc.fz_gemm_tc_check(_p(a), _p(w), c_int(m), c_int(w.shape[0]), c_int(k)) != 0:
            return False
        self._want(a, "linear input", (torch.bfloat16,), 2)
        self._want(w, "linear weight", (torch.bfloat16,), 2)
        self._want(cos, "cos table", (torch.float32,), 2)
        self._want(sin, "sin table", (torch.float32,), 2)
        self._want(q_out, "q", (torch.bfloat16,), 2)
        if bias is not None:
            self._want(bias, "linear bias", (torch.float32,), 1)
        n = (num_heads + 2 * num_kv_heads) * head_dim
        if w.shape != (n, k) or q_out.shape != (m, num_heads * head_dim) or cos.shape[1] != head_dim // 2 \
                or sin.shape != cos.shape or (bias is not None and bias.shape[0] != n):
            raise KernelError(f"linear_rope_kv_write: a {tuple(a.shape)}, w {tuple(w.shape)}, q {tuple(q_out.shape)}, "
                              f"cos {tuple(cos.shape)}")
        kp, vp, page_stride = self._pool(cache, num_kv_heads, head_dim)
        table = meta.table(cache.group)
        self._check(self.tc.fz_gemm_tc_qkv_rope(
            _p(a), _p(w), _p(bias), c_int(m), c_int(k), _p(cos), _p(sin), _p(meta.pos), _p(meta.seq_row), _p(table),
            c_int(table.shape[1]), _p(kp), _p(vp), c_longlong(page_stride), c_int(cache.page_size),
            c_int(1 if cache.write else 0), _p(q_out), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim),
            c_int(cos.shape[0]), _p(self.err), self._stream()), "linear_rope_kv_write (tensor cores)",
            ideal_linear_bytes(m, n, k, 2, 2, 2))
        return True

    def linear_argmax(self, a, w, bias, out) -> bool:
        m, k = a.shape
        n = w.shape[0]
        if not (self.use_tensor_cores and self.fuse_argmax and self.dtype == torch.bfloat16) or \
                self.tc.fz_gemm_tc_argmax_check(c_int(m), c_int(n), c_int(k)) != 0 or \
                self.tc.fz_gemm_tc_check(_p(a), _p(w), c_int(m), c_int(n), c_int(k)) != 0:
            return False
        self._want(a, "linear input", (torch.bfloat16,), 2)
        self._want(w, "linear weight", (torch.bfloat16,), 2)
        self._want(out, "argmax output", (torch.int32,), 1)
        if bias is not None:
            self._want(bias, "linear bias", (torch.float32,), 1)
        if w.shape[1] != k or out.shape[0] != m or (bias is not None and bias.shape[0] != n):
            raise KernelError(f"linear_argmax: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
        need = m * ((n + 127) // 128)
        tile_val = self._scratch("lm_head tile maxima", need, torch.float32)
        tile_idx = self._scratch("lm_head tile indices", need, torch.int32)
        self._check(self.tc.fz_gemm_tc_argmax(_p(a), _p(w), _p(bias), c_int(m), c_int(n), c_int(k), _p(tile_val),
                                              _p(tile_idx), _p(out), _p(self.err), self._stream()),
                    "linear_argmax (tensor cores)", ideal_linear_bytes(m, n, k, 2, 2, 0))
        self.launches += 1     # the reduction over the tiles
        return True

    def paged_attention(self, q, cache, meta, out, num_heads, num_kv_heads, head_dim, scale, window) -> None:
        self._want(q, "q", (self.dtype,), 2)
        self._want(out, "attention output", (self.dtype,), 2)
        n = q.shape[0]
        if q.shape[1] != num_heads * head_dim or out.shape != q.shape:
            raise KernelError(f"paged_attention: q {tuple(q.shape)}, out {tuple(out.shape)}")
        k, v, page_stride = self._pool(cache, num_kv_heads, head_dim)
        table = meta.table(cache.group)
        self._attention(q, k, v, page_stride, cache, meta, table, out, n, num_heads, num_kv_heads, head_dim, scale, window)

    def _attention(self, q, k, v, page_stride, cache, meta, table, out, n, hq, hkv, hd, scale, window) -> None:
        # least bytes: keys and values (a short row reads every key it sees; the rows of a long portion share them, so its
        # keys count once), the queries and the output
        kv = kv_tiles = 0
        if self._profile is not None:
            segs = list(getattr(meta, "segments", ()))
            key_bytes = hkv * hd * 2 * k.element_size()
            kv = contexts([sg for sg in segs if sg.n < LONG_PORTION]) * key_bytes + 2 * n * hq * hd * q.element_size()
            kv_tiles = sum(sg.pos0 + sg.n for sg in segs if sg.n >= LONG_PORTION) * key_bytes
        if self.use_tensor_cores and self.tc.fz_attn_decode_check(c_int(hq), c_int(hkv), c_int(hd)) == 0:
            plan = meta.plan
            if plan is None:
                raise KernelError("paged_attention: the step was not planned (plan_step with the need 'attention')")
            if plan.n_short_rows > 0:
                # rows of short portions and decoded tokens: split over key partitions, partials in float32 scratch
                parts = self.tc.fz_attn_partitions(c_int(meta.max_context))
                need = n * hq * parts * (hd + 2)
                part_o = self._scratch("attention partials", need, torch.float32)
                part_ml = part_o[n * hq * parts * hd:]
                self._check(self.tc.fz_attn_decode(
                    _p(q), _p(k), _p(v), _p(meta.pos), _p(meta.seq_row), _p(meta.seg), _p(table), c_int(table.shape[1]),
                    c_longlong(page_stride), c_int(cache.page_size), _p(out), _p(part_o), _p(part_ml), c_int(n),
                    c_int(hq), c_int(hkv), c_int(hd), c_float(scale), c_int(window), c_int(meta.max_context),
                    c_int(LONG_PORTION), c_int(1 if plan.single_tokens else 0), c_int(k.shape[0]), _p(self.err), self._stream()),
                    "paged_attention (decode)", kv)
                self.launches += 1    # the combine kernel
            if plan.n_tiles > 0 and self.prefill_tcgen05 and \
                    self.tc.fz_attn_prefill_tc_check(c_int(hq), c_int(hkv), c_int(hd), c_int(cache.page_size)) == 0:
                # rows of long portions on the tcgen05 flash-attention kernel; the pieces of tiles that the plan cut along
                # the keys leave partial results in float32 scratch (a slot per piece and head), merged by a second kernel
                piece_o = piece_ml = None
                if plan.n_cuts > 0:
                    rows = plan.n_pieces * hq * TILE_ROWS
                    piece_o = self._scratch("prefill pieces", rows * (hd + 2), torch.float32)
                    piece_ml = piece_o[rows * hd:]
                self._check(self.tc.fz_attn_prefill_tc(
                    _p(q), c_int(n), _p(k), _p(v), c_longlong(page_stride), c_int(k.shape[0]), _p(meta.seg), _p(plan.tiles),
                    c_int(plan.n_tiles), _p(plan.cuts), c_int(plan.n_cuts), _p(piece_o), _p(piece_ml), _p(table),
                    c_int(table.shape[1]), c_int(cache.page_size), _p(out), c_int(hq),
                    c_int(hkv), c_int(hd), c_float(scale), c_int(window), _p(self.err), self._stream()),
                    "paged_attention (prefill, tcgen05)", kv_tiles)
                if plan.n_cuts > 0:
                    self.launches += 1    # the merge kernel
            elif plan.n_tiles > 0 and plan.n_cuts > 0:
                raise KernelError("paged_attention: the step's tiles are cut along the keys, which only the tcgen05 kernel takes")
            elif plan.n_tiles > 0:
                self._check(self.tc.fz_attn_prefill(
                    _p(q), _p(k), _p(v), _p(meta.seg), _p(plan.tiles), c_int(plan.n_tiles), _p(table),
                    c_int(table.shape[1]), c_longlong(page_stride), c_int(cache.page_size), _p(out), c_int(hq),
                    c_int(hkv), c_int(hd), c_float(scale), c_int(window), self._stream()), "paged_attention (prefill)")
            return
        self._check(self.core.fz_attn_simt(
            _p(q), _p(k), _p(v), _p(meta.pos), _p(meta.seq_row), _p(table), c_int(table.shape[1]),
            c_longlong(page_stride), c_int(cache.page_size), _p(out), c_int(_CODE[self.dtype]), c_int(n), c_int(hq),
            c_int(hkv), c_int(hd), c_float(scale), c_int(window), _p(self.err), self._stream()), "paged_attention", kv)

    def swiglu(self, gate_up, out) -> None:
        self._want(gate_up, "gate_up", (self.dtype,), 2)
        self._want(out, "swiglu output", (self.dtype,), 2)
        n, i = out.shape
        if gate_up.shape != (n, 2 * i):
            raise KernelError(f"swiglu: gate_up {tuple(gate_up.shape)}, out {tuple(out.shape)}")
        self._check(self.core.fz_swiglu(_p(gate_up), _p(out), c_int(_CODE[self.dtype]), c_int(n), c_int(i),
                                        self._stream()), "swiglu")

    def argmax(self, logits, out) -> None:
        self._want(logits, "logits", (torch.float32,), 2)
        self._want(out, "argmax output", (torch.int32,), 1)
        r, v = logits.shape
        if out.shape[0] != r:
            raise KernelError(f"argmax: logits {tuple(logits.shape)}, out {tuple(out.shape)}")
        # scratch of the row-split argmax: per row up to S partial (value, index) pairs and one counter (kept zero)
        cap, slices = max(r, 64), int(self.core.fz_argmax_max_slices())
        pv = self._scratch("argmax partial values", cap * slices, torch.float32)
        pi = self._scratch("argmax partial indices", cap * slices, torch.int32)
        cnt = self._scratch("argmax counters", cap, torch.int32, zero=True)
        self._check(self.core.fz_argmax(_p(logits), _p(out), c_int(r), c_int(v), _p(pv), _p(pi), _p(cnt), self._stream()),
                    "argmax")

    def sample(self, logits, temperature, uniform, out) -> None:
        self._want(logits, "logits", (torch.float32,), 2)
        self._want(temperature, "temperature", (torch.float32,), 1)
        self._want(uniform, "uniform", (torch.float64,), 1)
        self._want(out, "sample output", (torch.int32,), 1)
        r, v = logits.shape
        if out.shape[0] != r or temperature.shape[0] != r or uniform.shape[0] != r:
            raise KernelError("sample: row counts differ")
        self._check(self.core.fz_sample(_p(logits), _p(temperature), _p(uniform), _p(out), c_int(r), c_int(v),
                                        self._stream()), "sample")

    def sample_filtered(self, logits, temperature, top_k, top_p, uniform, out) -> None:
        self._want(logits, "logits", (torch.float32,), 2)
        self._want(temperature, "temperature", (torch.float32,), 1)
        self._want(top_k, "top_k", (torch.int32,), 1)
        self._want(top_p, "top_p", (torch.float32,), 1)
        self._want(uniform, "uniform", (torch.float64,), 1)
        self._want(out, "sample output", (torch.int32,), 1)
        r, v = logits.shape
        if any(t.shape[0] != r for t in (out, temperature, top_k, top_p, uniform)):
            raise KernelError("sample_filtered: row counts differ")
        weights = self._scratch("sampling weights", r * v, torch.float64)       # exp(x / T - max) of every token
        self._check(self.core.fz_sample_filtered(_p(logits), _p(temperature), _p(top_k), _p(top_p), _p(uniform), _p(weights),
                                                 _p(out), c_int(r), c_int(v), self._stream()), "sample_filtered")
