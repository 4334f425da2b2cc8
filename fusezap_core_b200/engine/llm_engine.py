"""LLMEngine: requests in, tokens out, by continuous batching over the paged cache.

The Python entry point, with the reference's names (fusezap/serve/engine.py:1-8, 366-369, 542-563, 750-763):

  model = load_model(path, dtype="bfloat16", device="cuda:0", max_len=4096)
  eng = LLMEngine(model, num_blocks=1024, block_size=16, max_num_seqs=32)
  rid = eng.add_request(prompt_ids, SamplingParams(max_tokens=64))
  while eng.has_unfinished():
      for out in eng.step():          # a RequestOutput per request that got a token (or finished) in this step
          ...
  eng.generate(prompts, params)       # runs prompts to the end, returns each one's new tokens

A step is: schedule -> pack the batch's int32 metadata in pinned memory -> one host-to-device copy -> the model's step
function -> device sampling -> one device-to-host copy of the chosen ids -> emit. Decode-only steps replay a CUDA graph
captured per batch-size bucket (1, 2, 4, ... max_num_seqs), so their cost on the host is one copy and one launch; and
while requests only decode, the next step is launched (fed from the ids still on the device) before the host reads the
last one's tokens, so the device does not idle between steps.
"""
from __future__ import annotations
import itertools
from dataclasses import dataclass
from typing import Iterable, Sequence as Seq

import numpy as np
import torch

from ..cache import CacheManager
from ..sampling import RequestSampler, SamplingParams
from .model import DecoderModel
from .scheduler import Scheduler, SchedulerConfig, SchedulerOutput, Sequence, SeqStatus
from .step import Portion, StepRunner


@dataclass
class RequestOutput:
    request_id: int
    new_token_ids: list[int]
    token_ids: list[int]
    finished: bool = False
    finish_reason: str | None = None      # "stop" | "length" | "abort"
    num_prompt_tokens: int = 0


@dataclass
class _Launched:
    """A step that is on the stream and whose tokens the host has not read yet."""
    rows: list            # (request, index of its token among the step's chosen ids), for every request that gets one
    slot: int             # which of the two pinned id buffers the ids arrive in
    logits: torch.Tensor | None
    event: "torch.cuda.Event | None"
    all_produce: bool     # every running request gets a token from this step


class LLMEngine:
    def __init__(self, model: DecoderModel, num_blocks: int = 1024, block_size: int = 16, max_num_seqs: int = 32,
                 max_prefill_tokens: int | None = None, max_model_len: int | None = None,
                 max_num_batched_tokens: int | None = None, prefill_first: int = 0, cuda_graphs: bool = True, lookahead: bool = True,
                 graph_rows: int = 256):
        self.model = model
        self.max_model_len = int(max_model_len or model.max_len)
        if self.max_model_len > model.max_len:
            raise ValueError(f"max_model_len {self.max_model_len} exceeds the length the model was loaded for ({model.max_len})")
        max_prefill_tokens = int(max_prefill_tokens or min(2048, self.max_model_len))
        self.cfg = SchedulerConfig(max_num_seqs, max_prefill_tokens, max_num_batched_tokens, prefill_first)
        dev = model.device
        self.cache = CacheManager(model.cache_needs(), model.state_needs(), block_size, num_blocks, max_num_seqs,
                                  self.max_model_len, model.ops.dtype, dev)
        self.scheduler = Scheduler(self.cfg, self.cache)
        rows = self.cfg.token_budget
        self.runner = StepRunner(model, self.cache, max_rows=rows, max_wanted=max_num_seqs, max_segments=max_num_seqs)
        self.ops = model.ops
        self.stop_ids = set(model.spec.eos_token_ids)
        self.seqs: dict[int, Sequence] = {}
        self._ids, self._arrival = itertools.count(), itertools.count()
        pin = dev.type == "cuda"
        R = max_num_seqs
        # per-step sampling inputs and outputs: pinned on the host, fixed buffers on the device
        # (two of each host buffer: a step may be launched while the one before it is still in flight)
        self._temp_h = torch.zeros(2, R, dtype=torch.float32, pin_memory=pin)
        self._unif_h = torch.zeros(2, R, dtype=torch.float64, pin_memory=pin)
        self._topk_h = torch.zeros(2, R, dtype=torch.int32, pin_memory=pin)
        self._topp_h = torch.ones(2, R, dtype=torch.float32, pin_memory=pin)
        self._ids_h = torch.zeros(2, R, dtype=torch.int32, pin_memory=pin)
        self._events = [torch.cuda.Event() for _ in range(2)] if pin else None
        self._slot = 0
        self._pending: _Launched | None = None
        self.lookahead = bool(lookahead)
        self._temp_d = torch.zeros(R, dtype=torch.float32, device=dev)
        self._unif_d = torch.zeros(R, dtype=torch.float64, device=dev)
        self._topk_d = torch.zeros(R, dtype=torch.int32, device=dev)
        self._topp_d = torch.ones(R, dtype=torch.float32, device=dev)
        self._ids_d = torch.zeros(R, dtype=torch.int32, device=dev)
        self.runner.prev_ids = self._ids_d
        self.cuda_graphs = bool(cuda_graphs) and pin and model.graph_safe()
        # Captured steps. Decode steps: by (padded row count, how the tokens are chosen). Other steps of at most
        # `graph_rows` rows (portions of prompts, with or without decoded tokens beside them) are bound by the host's
        # launches, not by the GPU: they are captured too, by the sizes that fix their launches, the second time such
        # a step comes up (all else a step depends on lies in device memory at fixed addresses).
        self.graph_rows = int(graph_rows)
        self._step_seen: dict[tuple, int] = {}
        self._step_keys: list[tuple] = []                        # captured non-decode steps, oldest first
        self._graphs: dict[tuple, torch.cuda.CUDAGraph] = {}     # key -> captured step
        self.launches_per_graph: dict[tuple, int] = {}           # kernels of this package in one replay of it
        self._greedy_step = True
        self._ids_only = False
        self._filtered_step = False
        self._buckets = sorted({min(1 << i, R) for i in range(R.bit_length() + 1)})
        self.stats = {"steps": 0, "decode_steps": 0, "prefill_steps": 0, "mixed_steps": 0, "tokens": 0,
                      "preemptions": 0, "graph_replays": 0, "step_graph_replays": 0, "lookahead_steps": 0, "h2d_bytes": 0, "d2h_bytes": 0}

    # ---- a model and its engine in one call
    @classmethod
    def from_pretrained(cls, path: str, dtype: str = "bfloat16", device: str = "cuda:0", max_model_len: int = 2048,
                        ops=None, **engine_options) -> "LLMEngine":
        """`load_model(path, dtype, device, max_len=max_model_len)` and an engine over it; `engine_options` are the
        constructor's (num_blocks, block_size, max_num_seqs, ...)."""
        from .model import load_model
        model = load_model(path, dtype, device, max_len=max_model_len, ops=ops)
        return cls(model, max_model_len=max_model_len, **engine_options)

    @classmethod
    def from_random(cls, config: dict | str, seed: int = 0, dtype: str = "bfloat16", device: str = "cuda:0",
                    max_model_len: int = 2048, ops=None, **engine_options) -> "LLMEngine":
        """An engine over a model with seeded random weights drawn on the device. `config`: a config.json dictionary, or
        the name of a preset of this package (`tiny-llama`, `llama-3.1-8b`, ...)."""
        from .model import random_model
        if isinstance(config, str):
            from ..cli import load_preset
            config = load_preset(config)
        model = random_model(config, dtype, device, seed=seed, max_len=max_model_len, ops=ops)
        return cls(model, max_model_len=max_model_len, **engine_options)

    # ---- requests
    def add_request(self, prompt_ids: Seq[int], params: SamplingParams | None = None, request_id: int | None = None) -> int:
        params = params or SamplingParams()
        rid = next(self._ids) if request_id is None else request_id
        if rid in self.seqs:
            raise ValueError(f"request id {rid} is in use")
        if len(prompt_ids) + params.max_tokens > self.max_model_len:
            raise ValueError(f"prompt ({len(prompt_ids)}) + max_tokens ({params.max_tokens}) exceeds max_model_len {self.max_model_len}")
        vocab = self.model.spec.vocab_size
        prompt = [int(t) for t in prompt_ids]
        if any(t < 0 or t >= vocab for t in prompt):
            raise ValueError(f"a prompt token lies outside the vocabulary of {vocab}")
        seq = Sequence(rid, prompt, params, arrival=next(self._arrival))
        seq.sampler = RequestSampler(params)
        self.scheduler.add(seq, params.max_tokens)
        self.seqs[rid] = seq
        return rid

    def abort(self, request_id: int) -> RequestOutput | None:
        seq = self.seqs.get(request_id)
        if seq is None or seq.status == SeqStatus.FINISHED:
            return None
        self.scheduler.finish(seq, "abort")
        return self._out(seq, [])

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished()

    def release(self, request_id: int) -> None:
        s = self.seqs.get(request_id)
        if s is not None and s.status == SeqStatus.FINISHED:
            del self.seqs[request_id]

    def _out(self, seq: Sequence, new: list[int]) -> RequestOutput:
        return RequestOutput(seq.seq_id, new, list(seq.output), seq.status == SeqStatus.FINISHED, seq.finish_reason,
                             len(seq.prompt))

    # ---- one step
    def step(self) -> list[RequestOutput]:
        """Completes one model step and returns its tokens. With `lookahead`, the step after it is launched first
        whenever it is certain what it holds (see `_speculate`), so the device never waits for the host between
        decode steps."""
        cur, self._pending = self._pending, None
        if cur is not None and not any(s.status == SeqStatus.RUNNING for s, _ in cur.rows):
            cur = None            # launched ahead for requests that have all ended since: nothing to read from it
        if cur is None:
            so = self.scheduler.schedule()
            self.stats["preemptions"] += len(so.preempted)
            if so.empty:
                return []
            portions, owners = self._portions(so)
            rows = [(s, i) for i, s in enumerate(s for s, p in zip(owners, portions) if p.want)]
            kind = "decode_steps" if not so.prefill else "prefill_steps" if not so.decode else "mixed_steps"
            cur = self._launch(portions, rows, decode_only=not so.prefill,
                               all_produce=len(rows) == len(self.scheduler.running), kind=kind)
        nxt = self._speculate(cur) if self.lookahead else None
        outs = self._complete(cur)
        self._pending = nxt
        return outs

    def _speculate(self, cur: "_Launched") -> "_Launched | None":
        """Launches the decode step that follows `cur` before cur's tokens are known to the host: each row takes its
        token from the ids cur leaves on the device. Only when that step is certain: nothing waits for admission, every
        running request gets a token from cur, all of them are sampled on the device, and the pages are there. A request
        that cur ends by length is left out; one that cur ends by a stop token runs one token too many, which
        `_complete` drops (its pages are given back in stream order, so nobody reads what it wrote)."""
        sch, cache = self.scheduler, self.cache
        if sch.waiting or not cur.all_produce or not cur.rows:
            return None
        rows = []
        for seq, i in cur.rows:
            p = seq.params
            if seq.status != SeqStatus.RUNNING or not p.on_device:
                return None
            if len(seq.output) + 1 >= p.max_tokens or seq.num_tokens + 1 >= self.max_model_len:
                continue
            rows.append((seq, i))
        if not rows or len(rows) > self.cfg.token_budget:
            return None
        # the pages of all rows together: count them before taking any
        need = [0] * len(cache.groups)
        for seq, _ in rows:
            for g, n in enumerate(cache.pages_needed(seq.seq_id, seq.num_computed + 1)):
                need[g] += n
        if any(n > g.allocator.num_free for n, g in zip(need, cache.groups)):
            return None
        portions = []
        for seq, i in rows:
            cache.ensure(seq.seq_id, seq.num_computed + 1)
            portions.append(Portion(seq.seq_id, [0], [0], src=i))
        sch.steps += 1
        self.stats["lookahead_steps"] += 1
        return self._launch(portions, [(s, j) for j, (s, _) in enumerate(rows)], decode_only=True, all_produce=True)

    def _complete(self, cur: "_Launched") -> list[RequestOutput]:
        st = self.stats
        if cur.event is not None:
            cur.event.synchronize()
        self.ops.check_errors(copied=True)
        ids = self._ids_h[cur.slot].numpy()
        outs = []
        for seq, i in cur.rows:
            if seq.status != SeqStatus.RUNNING:        # aborted meanwhile, or ended by the step before
                continue
            if seq.params.on_device:
                tok = int(ids[i])
            else:
                row = cur.logits[i].detach().to("cpu", torch.float32).numpy()
                st["d2h_bytes"] += row.nbytes
                tok = seq.sampler.host_choice(row, seq.tokens)
            outs.append(self._emit(seq, tok))
        return outs

    def _portions(self, so: SchedulerOutput) -> tuple[list[Portion], list[Sequence]]:
        portions, owners = [], []
        for seq in so.decode:
            portions.append(Portion(seq.seq_id, [seq.token_at(seq.num_computed)], [0]))
            owners.append(seq)
        for seq, start, n in so.prefill:
            toks = seq.tokens_between(start, start + n)
            portions.append(Portion(seq.seq_id, toks, [n - 1] if start + n == seq.num_tokens else []))
            owners.append(seq)
        return portions, owners

    def _launch(self, portions, rows, decode_only: bool, all_produce: bool, kind: str = "decode_steps") -> "_Launched":
        """Puts one step on the stream: metadata and sampling inputs up, the model's step, the choice of tokens, the
        ids and the error word down. Does not wait for it."""
        runner, ops, st = self.runner, self.ops, self.stats
        slot = self._slot = (self._slot + 1) % 2
        temp_h, unif_h, topk_h, topp_h = self._temp_h[slot], self._unif_h[slot], self._topk_h[slot], self._topp_h[slot]
        R = len(rows)
        filtered = False
        for seq, i in rows:
            p = seq.params
            device_row = p.on_device and not p.greedy
            temp_h[i] = p.temperature if device_row else 0.0
            unif_h[i] = seq.sampler.next_uniform() if device_row else 0.0
            topk_h[i] = p.top_k if device_row else 0
            topp_h[i] = p.top_p if device_row else 1.0
            filtered = filtered or (device_row and p.filtered)
        # all rows greedy: the row-split argmax kernel picks the tokens; else a sampling kernel (argmax for its greedy
        # rows): the plain one, or the one with the top-k and top-p filters if some row has them
        self._greedy_step = all(s.params.greedy or not s.params.on_device for s, _ in rows)
        self._ids_only = all(s.params.greedy and s.params.on_device for s, _ in rows)
        self._filtered_step = filtered
        bucket = next((b for b in self._buckets if b >= len(portions)), None) if decode_only and self.cuda_graphs else None
        pad = bucket or 0
        starts = runner.prepare(portions, pad_rows=pad, pad_wanted=pad)
        key = None
        if bucket is not None:
            key = (bucket, self._greedy_step, self._ids_only, self._filtered_step)
        elif self.cuda_graphs and runner.meta.n_rows <= self.graph_rows:
            m = runner.meta
            sig = ("step", m.n_rows, m.n_wanted, m.n_tiles, m.n_short_rows > 0, self._greedy_step, self._ids_only,
                   self._filtered_step)
            if len(self._step_seen) > 4096:
                self._step_seen.clear()
            self._step_seen[sig] = self._step_seen.get(sig, 0) + 1
            if sig in self._graphs or self._step_seen[sig] >= 2:
                key = sig
        if key is not None:
            # a captured step must cover every context it may be replayed with (its launch sizes are fixed)
            runner.meta.max_context = self.max_model_len
        n_w = runner.meta.n_wanted
        if n_w:
            temp_h[R:n_w] = 0.0
            self._temp_d[:n_w].copy_(temp_h[:n_w], non_blocking=True)
            self._unif_d[:n_w].copy_(unif_h[:n_w], non_blocking=True)
            if filtered:
                topk_h[R:n_w] = 0
                topp_h[R:n_w] = 1.0
                self._topk_d[:n_w].copy_(topk_h[:n_w], non_blocking=True)
                self._topp_d[:n_w].copy_(topp_h[:n_w], non_blocking=True)
        st["h2d_bytes"] += runner.meta.size * 4 + n_w * (20 if filtered else 12)
        if key is not None:
            g = self._graphs.get(key)
            if g is None:
                # warm-up (builds, sets kernel attributes, sizes the buffers) on a copy of the ids the step may read
                keep = self._ids_d.clone()
                self._eager(n_w)
                torch.cuda.synchronize()
                self._ids_d.copy_(keep)
                g = torch.cuda.CUDAGraph()
                before = ops.launches
                with torch.cuda.graph(g):
                    self._eager(n_w)
                self.launches_per_graph[key] = ops.launches - before
                self._graphs[key] = g
                if key[0] == "step":
                    self._step_keys.append(key)
                    if len(self._step_keys) > 64:      # the oldest goes, once nothing of it is in flight
                        torch.cuda.synchronize()
                        old = self._step_keys.pop(0)
                        del self._graphs[old], self.launches_per_graph[old]
            g.replay()
            ops.launches += self.launches_per_graph[key]
            st["graph_replays"] += 1
            if key[0] == "step":
                st["step_graph_replays"] += 1
            logits = None if self._ids_only else runner.ws.get("logits", (n_w, self.model.spec.vocab_size), torch.float32)
        else:
            logits = self._eager(n_w)
        runner.commit(portions, starts)
        n_tokens = 0
        for p, s in zip(portions, starts):
            self.seqs[p.req].num_computed = s + len(p.tokens)
            n_tokens += len(p.tokens)
        if n_w:
            self._ids_h[slot][:n_w].copy_(self._ids_d[:n_w], non_blocking=True)
        ops.errors_to_host()
        event = None
        if self.model.device.type == "cuda":
            event = self._events[slot]
            event.record(torch.cuda.current_stream(self.model.device))
        st["d2h_bytes"] += n_w * 4 + 4
        st["steps"] += 1
        st["tokens"] += n_tokens
        st[kind] += 1
        return _Launched(rows, slot, logits, event, all_produce)

    def _eager(self, n_wanted: int) -> torch.Tensor | None:
        # a step whose rows are all greedy and picked on the device needs no logits: the lm_head product may then keep
        # only the largest value of every row
        ids_only = n_wanted > 0 and self._ids_only
        logits = self.runner.forward(self._ids_d[:n_wanted] if ids_only else None)
        if logits is None:
            return None
        if n_wanted and self._greedy_step:
            self.ops.argmax(logits, self._ids_d[:n_wanted])
        elif n_wanted and self._filtered_step:
            self.ops.sample_filtered(logits, self._temp_d[:n_wanted], self._topk_d[:n_wanted], self._topp_d[:n_wanted],
                                     self._unif_d[:n_wanted], self._ids_d[:n_wanted])
        elif n_wanted:
            self.ops.sample(logits, self._temp_d[:n_wanted], self._unif_d[:n_wanted], self._ids_d[:n_wanted])
        return logits

    def _emit(self, s: Sequence, tok: int) -> RequestOutput:
        s.output.append(tok)
        p = s.params
        if (not p.ignore_eos and tok in self.stop_ids) or tok in p.stop_token_ids:
            self.scheduler.finish(s, "stop")
        elif len(s.output) >= p.max_tokens or s.num_tokens >= self.max_model_len:
            self.scheduler.finish(s, "length")
        return self._out(s, [tok])

    # ---- convenience
    def generate(self, prompts: Iterable[Seq[int]], params: SamplingParams | Seq[SamplingParams] | None = None,
                 max_steps: int | None = None) -> list[list[int]]:
        prompts = list(prompts)
        ps = list(params) if isinstance(params, (list, tuple)) else [params or SamplingParams()] * len(prompts)
        rids = [self.add_request(p, q) for p, q in zip(prompts, ps)]
        n = 0
        while any(self.seqs[r].status != SeqStatus.FINISHED for r in rids):
            self.step()
            n += 1
            if max_steps is not None and n > max_steps:
                raise RuntimeError(f"not finished after {max_steps} steps")
        res = [list(self.seqs[r].output) for r in rids]
        for r in rids:
            self.release(r)
        return res
