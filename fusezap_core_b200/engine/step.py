"""The step function: one batch of (request, its next tokens) through the model, from the cache, to logits.

A step takes any mix of prompt portions and single decoded tokens, cut anywhere. It runs only the tokens it is given:
each token's keys and values go into its request's pages, attention reads the earlier ones from there, and the logits
of the wanted rows come back as one float32 (R, vocab) tensor. The reference runs prompt portions and decoded tokens as
two fixed-shape forwards over one packed int32 upload (fusezap/serve/engine.py:137-203,
fusezap/serve/kv_cache.py:382-405, 471-513); here it is one forward of any shape.

Per step the host packs one int32 block and copies it to the device once:
  tokens[N] | pos[N] | seq_row[N] | src[N] | sel[R] | segments[S x 4] | one block table (S x MB) per cache group | extra
seq_row[n] is the row of the request's block table in this step (-1: padding row), sel the rows whose logits are
wanted (-1: none), a segment is (first row, rows, first position, state slot) of one request's portion. `extra` belongs
to the kernel table: the mixers of the model say what kinds of step data their kernels need (`Mixer.step_needs()`), the
table says how many int32 it wants for them (`Ops.step_extra_ints`) and fills them when the step is packed
(`Ops.plan_step`), before the one copy. The step function itself knows nothing of any kernel's tiling.
"""
from __future__ import annotations
from dataclasses import dataclass, field
from typing import Any, Hashable, Sequence

import numpy as np
import torch

from ..cache import CacheManager
from ..parts import LayerCache
from .model import DecoderModel



@dataclass
class Portion:
    """One request's next tokens in a step; `want`: places among these tokens whose logits are asked for."""
    req: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()
    src: int = -1      # >= 0 (single-token portions only): the token is the id the previous step chose for its wanted
                       # row `src`, taken on the device; `tokens` then only gives the count


@dataclass
class Segment:
    req: Hashable
    row0: int          # first row of the portion in the step
    n: int             # tokens in the portion
    pos0: int          # position of its first token
    seq_row: int       # row of its block tables in the step metadata
    state_slot: int    # per-request state slot (-1: the model keeps no state)


class Workspace:
    """Scratch buffers by name. A buffer is allocated once with `row_capacity` rows (grown only if a step is larger)
    and handed out as a view of the rows asked for, so a captured step always sees the same addresses."""
    def __init__(self, device: torch.device, row_capacity: int):
        self.device, self.row_capacity = device, row_capacity
        self._bufs: dict[tuple, torch.Tensor] = {}
        self._retired: list[torch.Tensor] = []      # outgrown buffers: a captured step may still point at them

    def get(self, tag: str, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        key = (tag, tuple(shape[1:]), dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.shape[0] < shape[0]:
            if buf is not None:
                self._retired.append(buf)
            buf = torch.empty((max(self.row_capacity, shape[0]), *shape[1:]), dtype=dtype, device=self.device)
            self._bufs[key] = buf
        return buf[:shape[0]]

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._bufs.values())


class StepMeta:
    """The step's int32 metadata: a pinned host block and its device copy with fixed offsets for a given capacity."""
    def __init__(self, device: torch.device, max_rows: int, max_wanted: int, max_segments: int, num_groups: int,
                 pages_per_request: int, extra_ints: int = 0):
        self.device = device
        self.max_rows, self.max_wanted, self.max_segments = max_rows, max_wanted, max_segments
        self.num_groups, self.mb = num_groups, pages_per_request
        o = 0
        self.o_tokens, o = o, o + max_rows
        self.o_pos, o = o, o + max_rows
        self.o_row, o = o, o + max_rows
        self.o_src, o = o, o + max_rows
        self.o_sel, o = o, o + max_wanted
        self.o_seg, o = o, o + 4 * max_segments
        self.o_tab, o = o, o + num_groups * max_segments * pages_per_request
        self.extra_ints = extra_ints
        self.o_extra, o = o, o + extra_ints
        self.size = o
        # a ring of pinned host blocks: a block is rewritten only after the copy that read it has finished
        pin = device.type == "cuda"
        self._hosts = [torch.zeros(self.size, dtype=torch.int32, pin_memory=pin) for _ in range(4 if pin else 1)]
        self._events = [torch.cuda.Event() if pin else None for _ in self._hosts]
        self._used = [False] * len(self._hosts)
        self._turn = 0
        self.host = self._hosts[0]
        self.np = self.host.numpy()
        self.dev = torch.zeros(self.size, dtype=torch.int32, device=device)
        # filled per step
        self.n_rows = self.n_wanted = self.n_segments = 0
        self.segments: list[Segment] = []
        self.max_context = 0      # the longest context (position + 1) among the step's rows
        self.page_size = 0        # of the cache the step was packed against
        self.max_portion = 0      # the longest portion
        self.plan = None          # whatever the kernel table's `plan_step` keeps about this step (launch sizes and the like)

    # device views (static addresses; sliced to the step's sizes)
    @property
    def tokens(self) -> torch.Tensor: return self.dev[self.o_tokens: self.o_tokens + self.n_rows]
    @property
    def pos(self) -> torch.Tensor: return self.dev[self.o_pos: self.o_pos + self.n_rows]
    @property
    def seq_row(self) -> torch.Tensor: return self.dev[self.o_row: self.o_row + self.n_rows]
    @property
    def src(self) -> torch.Tensor: return self.dev[self.o_src: self.o_src + self.n_rows]
    @property
    def sel(self) -> torch.Tensor: return self.dev[self.o_sel: self.o_sel + self.n_wanted]
    @property
    def seg(self) -> torch.Tensor: return self.dev[self.o_seg: self.o_seg + 4 * self.max_segments].view(self.max_segments, 4)
    @property
    def extra(self) -> torch.Tensor: return self.dev[self.o_extra: self.o_extra + self.extra_ints]
    @property
    def extra_host(self) -> np.ndarray: return self.np[self.o_extra: self.o_extra + self.extra_ints]
    def table(self, group: int) -> torch.Tensor:
        n = self.max_segments * self.mb
        return self.dev[self.o_tab + group * n: self.o_tab + (group + 1) * n].view(self.max_segments, self.mb)

    def fill(self, cache: CacheManager, portions: Sequence[Portion], starts: Sequence[int], pad_rows: int = 0,
             pad_wanted: int = 0, ops: Any = None, needs: tuple = ()) -> None:
        """Pack the step, let the kernel table `ops` plan it for the kinds of step data in `needs`, and copy it to the
        device."""
        self.pack(cache, portions, starts, pad_rows, pad_wanted)
        plan_step = getattr(ops, "plan_step", None)
        if plan_step is not None:
            plan_step(self, needs)
        self.upload()

    def pack(self, cache: CacheManager, portions: Sequence[Portion], starts: Sequence[int], pad_rows: int = 0,
             pad_wanted: int = 0) -> None:
        """Pack the step on the host. starts[i]: position of the first token of portions[i]. pad_rows / pad_wanted: run
        the step with at least this many rows / wanted rows (padding rows are inert), for fixed-shape replay."""
        self._turn = (self._turn + 1) % len(self._hosts)
        if self._used[self._turn] and self._events[self._turn] is not None:
            self._events[self._turn].synchronize()
        self.host = self._hosts[self._turn]
        a = self.np = self.host.numpy()
        n = sum(len(p.tokens) for p in portions)
        r = sum(len(p.want) for p in portions)
        n_rows, n_wanted = max(n, pad_rows), max(r, pad_wanted)
        if n_rows > self.max_rows or n_wanted > self.max_wanted or len(portions) > self.max_segments:
            raise ValueError(f"step of {n_rows} rows, {n_wanted} wanted, {len(portions)} requests exceeds the capacity "
                             f"({self.max_rows}, {self.max_wanted}, {self.max_segments})")
        tok, pos, row, src = (a[o: o + n_rows] for o in (self.o_tokens, self.o_pos, self.o_row, self.o_src))
        src[:] = -1
        sel = a[self.o_sel: self.o_sel + n_wanted]
        seg = a[self.o_seg: self.o_seg + 4 * self.max_segments].reshape(self.max_segments, 4)
        tok[n:], pos[n:], row[n:], sel[r:] = 0, 0, -1, -1
        seg[len(portions):] = 0
        self.segments = []
        self.page_size = cache.page_size
        at = w = 0
        self.max_context = self.max_portion = 0
        for s, (p, start) in enumerate(zip(portions, starts)):
            k = len(p.tokens)
            tok[at: at + k] = np.asarray(p.tokens, dtype=np.int64)
            if p.src >= 0:
                if k != 1:
                    raise ValueError(f"request {p.req!r}: only a single token can come from the previous step's ids")
                src[at] = p.src
            pos[at: at + k] = np.arange(start, start + k)
            row[at: at + k] = s
            for j in p.want:
                if not 0 <= j < k:
                    raise ValueError(f"request {p.req!r}: wanted place {j} is outside its {k} tokens")
                sel[w] = at + j
                w += 1
            slot = cache.state_slot(p.req)
            seg[s] = (at, k, start, slot)
            self.segments.append(Segment(p.req, at, k, start, s, slot))
            self.max_context = max(self.max_context, start + k)
            self.max_portion = max(self.max_portion, k)
            at += k
        for g in range(self.num_groups):
            t = a[self.o_tab + g * self.max_segments * self.mb: self.o_tab + (g + 1) * self.max_segments * self.mb]
            t = t.reshape(self.max_segments, self.mb)
            for s, p in enumerate(portions):
                row, used = cache.table_row(g, p.req)
                t[s, :used] = row[:used]
                t[s, used:] = -1
        self.n_rows, self.n_wanted, self.n_segments = n_rows, n_wanted, len(portions)
        self.plan = None

    def upload(self) -> None:
        """The one host-to-device copy of the step's metadata."""
        self.dev.copy_(self.host, non_blocking=True)
        if self._events[self._turn] is not None:
            self._events[self._turn].record()
            self._used[self._turn] = True


@dataclass
class StepContext:
    ops: Any
    ws: Workspace
    meta: StepMeta
    positions: dict[str, Any]
    model: DecoderModel


class StepRunner:
    """Owns the step's metadata and scratch buffers and runs the model over them."""
    def __init__(self, model: DecoderModel, cache: CacheManager, max_rows: int, max_wanted: int | None = None,
                 max_segments: int | None = None):
        self.model, self.cache, self.ops = model, cache, model.ops
        dev = model.device
        self.max_rows = max_rows
        # what kinds of step data the mixers' kernels need, and how many int32 the kernel table wants for them
        self.needs = tuple(sorted({k for e in model.spec.schedule for k in model.layers[e.layer].mixer.step_needs()}))
        max_segments = max_segments or max_rows
        extra = getattr(self.ops, "step_extra_ints", lambda *a: 0)(self.needs, max_rows, max_segments)
        self.meta = StepMeta(dev, max_rows, max_wanted or max_rows, max_segments, len(cache.groups),
                             cache.max_pages_per_request, extra)
        self.ws = Workspace(dev, max_rows)
        self.ctx = StepContext(self.ops, self.ws, self.meta, model.positions, model)
        self.prev_ids: torch.Tensor | None = None     # device int32: the ids the previous step chose (see Portion.src)
        self.layer_caches: list[LayerCache] = []
        for n, e in enumerate(model.spec.schedule):
            need = model.layers[e.layer].mixer.cache_need()
            lc = LayerCache(write=e.write_cache)
            if need is not None:
                g = cache.slot_group[e.cache]
                lc.keys, lc.values = cache.groups[g].view(e.cache)
                lc.group, lc.page_size = g, cache.page_size
            lc.state = {name: t for (entry, name), t in cache.states.tensors.items() if entry == n}
            self.layer_caches.append(lc)

    def forward(self, ids_out: torch.Tensor | None = None) -> torch.Tensor | None:
        """Runs the model over the metadata already filled; returns logits (n_wanted, vocab) float32. With `ids_out`
        (int32, n_wanted): if the kernel table can pick the largest logit of every wanted row without writing the logits
        out, it does, `ids_out` receives the token ids and None is returned; otherwise logits as usual."""
        model, ctx, meta = self.model, self.ctx, self.meta
        spec = model.spec
        begin, end = getattr(self.ops, "begin_step", None), getattr(self.ops, "end_step", None)
        if begin is not None:
            begin()
        try:
            return self._forward(model, ctx, meta, spec, ids_out)
        finally:
            if end is not None:
                end()

    def _forward(self, model, ctx, meta, spec, ids_out):
        x = self.ws.get("x", (meta.n_rows, spec.hidden_size), torch.float32)
        src = meta.src if self.prev_ids is not None else None
        if model.embed_scale != 1.0:
            self.ops.embed(model.embed, meta.tokens, x, src, self.prev_ids, model.embed_scale)
        else:
            self.ops.embed(model.embed, meta.tokens, x, src, self.prev_ids)
        delta = None
        for e, lc in zip(spec.schedule, self.layer_caches):
            x, delta = model.layers[e.layer].forward(ctx, x, delta, lc)
        logits = self.ws.get("logits", (meta.n_wanted, spec.vocab_size), torch.float32)
        if meta.n_wanted:
            h = model.final_norm.forward(ctx, x, delta, rows=meta.sel, n_rows=meta.n_wanted)
            transform = model.logit_transform
            fused = getattr(self.ops, "linear_argmax", None) if ids_out is not None and transform is None else None
            if fused is not None and fused(h, model.lm_head, None, ids_out):
                return None
            self.ops.linear(h, model.lm_head, None, logits)
            if transform is not None:
                transform.forward(ctx, logits)
        return logits

    def prepare(self, portions: Sequence[Portion], pad_rows: int = 0, pad_wanted: int = 0) -> list[int]:
        """Backs every portion with pages and packs the metadata. Returns each portion's first position."""
        cache = self.cache
        seen = set()
        starts = []
        for p in portions:
            if p.req in seen:
                raise ValueError(f"request {p.req!r} appears twice in one step")
            if len(p.tokens) == 0:
                raise ValueError(f"request {p.req!r} brings no tokens")
            seen.add(p.req)
            start = cache.computed.get(p.req, 0)
            cache.ensure(p.req, start + len(p.tokens))
            starts.append(start)
        self.meta.fill(cache, portions, starts, pad_rows, pad_wanted, self.ops, self.needs)
        return starts

    def commit(self, portions: Sequence[Portion], starts: Sequence[int]) -> None:
        for p, s in zip(portions, starts):
            self.cache.commit(p.req, s + len(p.tokens))

    def run(self, portions: Sequence[Portion]) -> torch.Tensor:
        starts = self.prepare(portions)
        logits = self.forward()
        self.commit(portions, starts)
        return logits
