"""LLMEngine: requests in, tokens out, by continuous batching over the paged cache.

The Python entry point, with the reference's names (fusezap/serve/engine.py:1-8, 366-369, 542-563, 750-763):

  model = load_model(path, dtype="bfloat16", device="cuda:0", max_len=4096)
  eng = LLMEngine(model, num_blocks=1024, block_size=16, max_num_seqs=32)     # or LLMEngine(model, EngineConfig(...))
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
from ..config import EngineConfig
from ..sampling import RequestSampler, SamplingParams
from .model import DecoderModel
from .request import Phase, Request
from .scheduler import Scheduler, StepPlan
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
    def __init__(self, model: DecoderModel, config: EngineConfig | None = None, **options):
        """`config`: the engine's options (`EngineConfig`); or give them as keywords (`num_blocks=..., block_size=...,
        max_num_seqs=..., max_prefill_tokens=..., max_model_len=...`, the reference's argument names), not both."""
        if config is not None and options:
            raise TypeError("give either an EngineConfig or options as keywords, not both")
        cfg = (config or EngineConfig(**options)).resolved(model.max_len)
        self.model, self.cfg = model, cfg
        self.max_model_len = cfg.max_model_len
        dev = model.device
        R = cfg.max_num_seqs
        self.cache = CacheManager(model.cache_needs(), model.state_needs(), cfg.block_size, cfg.num_blocks, R,
                                  self.max_model_len, model.ops.dtype, dev)
        self.scheduler = Scheduler(cfg, self.cache)
        self.runner = StepRunner(model, self.cache, max_rows=cfg.token_budget, max_wanted=R, max_segments=R)
        self.ops = model.ops
        self.stop_ids = set(model.spec.eos_token_ids)
        self.requests: dict[int, Request] = {}
        self._next_id, self._clock = itertools.count(), itertools.count()
        pin = dev.type == "cuda"
        # per-step sampling inputs and outputs: pinned on the host, fixed buffers on the device
        # (two of each host buffer: a step may be launched while the one before it is still in flight)
        self._temp_h = torch.zeros(2, R, dtype=torch.float32, pin_memory=pin)
        self._unif_h = torch.zeros(2, R, dtype=torch.float64, pin_memory=pin)
        self._topk_h = torch.zeros(2, R, dtype=torch.int32, pin_memory=pin)
        self._topp_h = torch.ones(2, R, dtype=torch.float32, pin_memory=pin)
        # (numpy views of the same pinned memory: writing an element of a tensor costs microseconds, of an array not)
        self._sampling_np = tuple(t.numpy() for t in (self._temp_h, self._unif_h, self._topk_h, self._topp_h))
        self._ids_h = torch.zeros(2, R, dtype=torch.int32, pin_memory=pin)
        self._events = [torch.cuda.Event() for _ in range(2)] if pin else None
        self._slot = 0
        self._pending: _Launched | None = None
        self.profile = bool(cfg.profile) and pin and hasattr(model.ops, "start_profile")
        self.lookahead = bool(cfg.lookahead) and not self.profile
        self._temp_d = torch.zeros(R, dtype=torch.float32, device=dev)
        self._unif_d = torch.zeros(R, dtype=torch.float64, device=dev)
        self._topk_d = torch.zeros(R, dtype=torch.int32, device=dev)
        self._topp_d = torch.ones(R, dtype=torch.float32, device=dev)
        self._ids_d = torch.zeros(R, dtype=torch.int32, device=dev)
        self.runner.prev_ids = self._ids_d
        self.cuda_graphs = bool(cfg.cuda_graphs) and pin and model.graph_safe() and not self.profile
        # Captured steps. Decode steps: by (padded row count, how the tokens are chosen). Other steps of at most
        # `graph_rows` rows (portions of prompts, with or without decoded tokens beside them) are bound by the host's
        # launches, not by the GPU: they are captured too, by the sizes that fix their launches, the second time such
        # a step comes up (all else a step depends on lies in device memory at fixed addresses).
        self.graph_rows = cfg.graph_rows
        self._step_seen: dict[tuple, int] = {}
        self._step_keys: list[tuple] = []                        # captured non-decode steps, oldest first
        self._graphs: dict[tuple, torch.cuda.CUDAGraph] = {}     # key -> captured step
        self.launches_per_graph: dict[tuple, int] = {}           # kernels of this package in one replay of it
        self._greedy_step = True
        self._ids_only = False
        self._filtered_step = False
        # row counts of the captured decode steps: powers of two, none above what a step can hold
        most = min(R, cfg.token_budget)
        self._buckets = sorted({min(1 << i, most) for i in range(most.bit_length() + 1)})
        self.stats = {"steps": 0, "decode_steps": 0, "prefill_steps": 0, "mixed_steps": 0, "tokens": 0,
                      "preemptions": 0, "graph_replays": 0, "step_graph_replays": 0, "lookahead_steps": 0, "h2d_bytes": 0, "d2h_bytes": 0}
        if self.profile:
            model.ops.start_profile()

    # ---- a model and its engine in one call
    @classmethod
    def from_pretrained(cls, path: str, dtype: str | None = None, device: str | None = None,
                        max_model_len: int | None = None, ops=None, config: EngineConfig | None = None,
                        **options) -> "LLMEngine":
        """`load_model(path, dtype, device, max_len=max_model_len)` and an engine over it. The options are
        `EngineConfig`'s, given as one object or as keywords (dtype, device, max_model_len, num_blocks, ...)."""
        from .model import load_model
        cfg = _config_from(config, dtype, device, max_model_len, options)
        model = load_model(path, cfg.dtype, cfg.device, max_len=cfg.max_model_len, ops=ops)
        return cls(model, cfg)

    @classmethod
    def from_random(cls, config_json: dict | str, seed: int = 0, dtype: str | None = None, device: str | None = None,
                    max_model_len: int | None = None, ops=None, config: EngineConfig | None = None,
                    **options) -> "LLMEngine":
        """An engine over a model with seeded random weights drawn on the device. `config_json`: a config.json
        dictionary, or the name of a preset of this package (`tiny-llama`, `llama-3.1-8b`, ...)."""
        from .model import random_model
        if isinstance(config_json, str):
            from ..cli import load_preset
            config_json = load_preset(config_json)
        cfg = _config_from(config, dtype, device, max_model_len, options)
        model = random_model(config_json, cfg.dtype, cfg.device, seed=seed, max_len=cfg.max_model_len, ops=ops)
        return cls(model, cfg)

    # ---- requests
    def add_request(self, prompt_ids: Seq[int], params: SamplingParams | None = None, request_id: int | None = None) -> int:
        """Queues a prompt (token ids); returns the request's id. Refuses an id in use, a prompt that cannot fit with
        its `max_tokens`, and token ids outside the vocabulary."""
        if params is None:
            params = SamplingParams()
        if request_id is None:
            request_id = next(self._next_id)
            while request_id in self.requests:
                request_id = next(self._next_id)
        elif request_id in self.requests:
            raise ValueError(f"request id {request_id} is in use")
        prompt = [int(t) for t in prompt_ids]
        room = self.max_model_len - len(prompt)
        if params.max_tokens > room:
            raise ValueError(f"prompt ({len(prompt)}) + max_tokens ({params.max_tokens}) exceeds max_model_len {self.max_model_len}")
        vocab = self.model.spec.vocab_size
        if prompt and not 0 <= min(prompt) <= max(prompt) < vocab:
            raise ValueError(f"a prompt token lies outside the vocabulary of {vocab}")
        req = Request(request_id, prompt, params, order=next(self._clock), sampler=RequestSampler(params))
        self.scheduler.submit(req)
        self.requests[request_id] = req
        return request_id

    def abort(self, request_id: int) -> RequestOutput | None:
        """Ends a request now; None if it is unknown or has ended."""
        req = self.requests.get(request_id)
        if req is None or req.phase is Phase.DONE:
            return None
        self.scheduler.retire(req, "abort")
        return self._report(req, ())

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished()

    def release(self, request_id: int) -> None:
        """Forgets a request that has ended (until then its tokens stay readable in `requests`)."""
        req = self.requests.get(request_id)
        if req is not None and req.phase is Phase.DONE:
            self.requests.pop(request_id)

    def _report(self, req: Request, new_tokens) -> RequestOutput:
        return RequestOutput(request_id=req.rid, new_token_ids=list(new_tokens), token_ids=list(req.generated),
                             finished=req.phase is Phase.DONE, finish_reason=req.ended_by,
                             num_prompt_tokens=len(req.prompt))

    # ---- one step
    def step(self) -> list[RequestOutput]:
        """Completes one model step and returns its tokens. With `lookahead`, the step after it is launched first
        whenever it is certain what it holds (see `_speculate`), so the device never waits for the host between
        decode steps."""
        cur, self._pending = self._pending, None
        if cur is not None and all(r.phase is not Phase.LIVE for r, _ in cur.rows):
            cur = None            # launched ahead for requests that have all ended since: nothing to read from it
        if cur is None:
            plan = self.scheduler.plan()
            self.stats["preemptions"] += len(plan.evicted)
            if plan.empty:
                return []
            portions, rows = self._portions(plan)
            n_decode = sum(1 for w in plan.work if w.decode)
            kind = "decode_steps" if n_decode == len(plan.work) else "mixed_steps" if n_decode else "prefill_steps"
            cur = self._launch(portions, rows, decode_only=n_decode == len(plan.work),
                               all_produce=len(rows) == len(self.scheduler.live), kind=kind)
        nxt = self._speculate(cur) if self.lookahead else None
        outs = self._complete(cur)
        self._pending = nxt
        return outs

    def _portions(self, plan: StepPlan) -> tuple[list[Portion], list[tuple[Request, int]]]:
        """The plan as the step function's portions, and (request, index among the step's chosen ids) for every
        request that gets a token from it: a request whose share reaches the end of what it knows."""
        portions, rows = [], []
        for w in plan.work:
            req, end = w.request, w.start + w.count
            last = end == req.known
            portions.append(Portion(req.rid, req.span(w.start, end), [w.count - 1] if last else []))
            if last:
                rows.append((req, len(rows)))
        return portions, rows

    def _speculate(self, cur: "_Launched") -> "_Launched | None":
        """Launches the decode step that follows `cur` before cur's tokens are known to the host: each row takes its
        token from the ids cur leaves on the device. Only when that step is certain: nothing waits for admission, every
        running request gets a token from cur, all of them are sampled on the device, and the pages are there. A request
        that cur ends by length is left out; one that cur ends by a stop token runs one token too many, which
        `_complete` drops (its pages are given back in stream order, so nobody reads what it wrote)."""
        sch, cache = self.scheduler, self.cache
        if sch.queue or not cur.all_produce or not cur.rows:
            return None
        rows = []
        for req, i in cur.rows:
            p = req.params
            if req.phase is not Phase.LIVE or not p.on_device:
                return None
            if len(req.generated) + 1 >= p.max_tokens or req.known + 1 >= self.max_model_len:
                continue
            rows.append((req, i))
        if not rows or len(rows) > self.cfg.token_budget:
            return None
        # the pages of all rows together: count them before taking any
        need = [0] * len(cache.groups)
        for req, _ in rows:
            for g, n in enumerate(cache.pages_needed(req.rid, req.cached + 1)):
                need[g] += n
        if any(n > g.allocator.num_free for n, g in zip(need, cache.groups)):
            return None
        portions = []
        for req, i in rows:
            cache.ensure(req.rid, req.cached + 1)
            portions.append(Portion(req.rid, [0], [0], src=i))
        sch.steps += 1
        self.stats["lookahead_steps"] += 1
        return self._launch(portions, [(r, j) for j, (r, _) in enumerate(rows)], decode_only=True, all_produce=True)

    def _complete(self, cur: "_Launched") -> list[RequestOutput]:
        st = self.stats
        if cur.event is not None:
            cur.event.synchronize()
        self.ops.check_errors(copied=True)
        ids = self._ids_h[cur.slot].numpy()
        outs = []
        for req, i in cur.rows:
            if req.phase is not Phase.LIVE:        # aborted meanwhile, or ended by the step before
                continue
            if req.params.on_device:
                tok = int(ids[i])
            else:
                row = cur.logits[i].detach().to("cpu", torch.float32).numpy()
                st["d2h_bytes"] += row.nbytes
                tok = req.sampler.host_choice(row, req.history)
            outs.append(self._take(req, tok))
        return outs

    def _launch(self, portions, rows, decode_only: bool, all_produce: bool, kind: str = "decode_steps") -> "_Launched":
        """Puts one step on the stream: metadata and sampling inputs up, the model's step, the choice of tokens, the
        ids and the error word down. Does not wait for it."""
        runner, ops, st = self.runner, self.ops, self.stats
        slot = self._slot = (self._slot + 1) % 2
        temp_h, unif_h, topk_h, topp_h = self._temp_h[slot], self._unif_h[slot], self._topk_h[slot], self._topp_h[slot]
        R = len(rows)
        filtered = False
        temp_a, unif_a, topk_a, topp_a = (a[slot] for a in self._sampling_np)
        temp_a[:R], unif_a[:R], topk_a[:R], topp_a[:R] = 0.0, 0.0, 0, 1.0      # greedy rows and rows sampled on the host
        for req, i in rows:
            p = req.params
            if p.on_device and not p.greedy:
                temp_a[i], unif_a[i], topk_a[i], topp_a[i] = p.temperature, req.sampler.next_uniform(), p.top_k, p.top_p
                filtered = filtered or p.filtered
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
            # a captured decode step must cover every context it may be replayed with (its launch sizes are fixed)
            runner.meta.max_context = self.max_model_len
        elif self.cuda_graphs and runner.meta.n_rows <= self.graph_rows:
            m = runner.meta
            # Other captured steps cover contexts up to the next power of two (at least 1,024) of the step's own, which is
            # part of their key: kernels size their scratch by rows x the context covered, and a step of a few hundred
            # rows sized for the whole `max_model_len` would hold hundreds of megabytes at long model lengths.
            covered = min(self.max_model_len, max(1024, 1 << (max(m.max_context, 1) - 1).bit_length()))
            sig = ("step", m.n_rows, m.n_wanted, covered, *getattr(ops, "step_signature", lambda _: ())(m), self._greedy_step,
                   self._ids_only, self._filtered_step)
            if len(self._step_seen) > 4096:
                self._step_seen.clear()
            self._step_seen[sig] = self._step_seen.get(sig, 0) + 1
            if sig in self._graphs or self._step_seen[sig] >= 2:
                key = sig
                m.max_context = covered
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
                # The first step of this shape runs kernel by kernel (which also builds what it needs, sets kernel
                # attributes and sizes the buffers) and is then recorded for the next one; recording launches nothing,
                # so the step runs exactly once (a part that updates per-request state in place is not advanced twice).
                logits = self._eager(n_w)
                g = torch.cuda.CUDAGraph()
                before = ops.launches
                with torch.cuda.graph(g):
                    self._eager(n_w)
                self.launches_per_graph[key] = ops.launches - before
                ops.launches = before
                self._graphs[key] = g
                if key[0] == "step":
                    self._step_keys.append(key)
                    if len(self._step_keys) > 64:      # the oldest goes, once nothing of it is in flight
                        torch.cuda.synchronize()
                        old = self._step_keys.pop(0)
                        del self._graphs[old], self.launches_per_graph[old]
            else:
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
            self.requests[p.req].cached = s + len(p.tokens)
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

    def _take(self, req: Request, tok: int) -> RequestOutput:
        """The request's next token has been chosen: keep it, and end the request if this token or its count says so."""
        req.generated.append(tok)
        p = req.params
        stops = tok in p.stop_token_ids or (tok in self.stop_ids and not p.ignore_eos)
        if stops:
            self.scheduler.retire(req, "stop")
        elif len(req.generated) >= p.max_tokens or req.known >= self.max_model_len:
            self.scheduler.retire(req, "length")
        return self._report(req, (tok,))

    # ---- convenience
    def generate(self, prompts: Iterable[Seq[int]], params: SamplingParams | Seq[SamplingParams] | None = None,
                 max_steps: int | None = None) -> list[list[int]]:
        """Runs the prompts to their ends; returns each one's new tokens, in the order of `prompts`. `params`: one for
        all, or one per prompt."""
        prompts = list(prompts)
        if isinstance(params, (list, tuple)):
            each = list(params)
            if len(each) != len(prompts):
                raise ValueError(f"{len(prompts)} prompts but {len(each)} sampling params")
        else:
            each = [params if params is not None else SamplingParams()] * len(prompts)
        mine = [self.requests[self.add_request(p, q)] for p, q in zip(prompts, each)]
        steps = 0
        while not all(r.phase is Phase.DONE for r in mine):
            if max_steps is not None and steps >= max_steps:
                raise RuntimeError(f"not finished after {max_steps} steps")
            self.step()
            steps += 1
        for r in mine:
            self.release(r.rid)
        return [list(r.generated) for r in mine]

    def profile_report(self) -> dict:
        """With `profile` on: per kernel class the launches and device time since the engine was made."""
        if not self.profile:
            raise RuntimeError("the engine was made without profile=True")
        return self.ops.profile_report()


def _config_from(config: EngineConfig | None, dtype, device, max_model_len, options: dict) -> EngineConfig:
    from ..config.engine_config import DEFAULT_MODEL_LEN
    given = {k: v for k, v in (("dtype", dtype), ("device", device), ("max_model_len", max_model_len)) if v is not None}
    if config is not None:
        if options or given:
            raise TypeError("give either an EngineConfig or options as keywords, not both")
        cfg = config
    else:
        cfg = EngineConfig(**given, **options)
    if cfg.max_model_len is None:
        import dataclasses
        cfg = dataclasses.replace(cfg, max_model_len=DEFAULT_MODEL_LEN)
    return cfg
