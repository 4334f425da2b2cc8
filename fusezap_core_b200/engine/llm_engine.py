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
captured per batch-size bucket (1, 2, 4, ... max_num_seqs), so their cost on the host is one copy and one launch.
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


class LLMEngine:
    def __init__(self, model: DecoderModel, num_blocks: int = 1024, block_size: int = 16, max_num_seqs: int = 32,
                 max_prefill_tokens: int | None = None, max_model_len: int | None = None,
                 max_num_batched_tokens: int | None = None, prefill_first: int = 0, cuda_graphs: bool = True):
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
        self._temp_h = torch.zeros(R, dtype=torch.float32, pin_memory=pin)
        self._unif_h = torch.zeros(R, dtype=torch.float64, pin_memory=pin)
        self._ids_h = torch.zeros(R, dtype=torch.int32, pin_memory=pin)
        self._temp_d = torch.zeros(R, dtype=torch.float32, device=dev)
        self._unif_d = torch.zeros(R, dtype=torch.float64, device=dev)
        self._ids_d = torch.zeros(R, dtype=torch.int32, device=dev)
        self.cuda_graphs = bool(cuda_graphs) and pin and model.graph_safe()
        self._graphs: dict[tuple, torch.cuda.CUDAGraph] = {}     # (bucket, all rows greedy) -> captured step
        self.launches_per_graph: dict[tuple, int] = {}           # kernels of this package in one replay of it
        self._greedy_step = True
        self._buckets = sorted({min(1 << i, R) for i in range(R.bit_length() + 1)})
        self.stats = {"steps": 0, "decode_steps": 0, "prefill_steps": 0, "mixed_steps": 0, "tokens": 0,
                      "preemptions": 0, "graph_replays": 0, "h2d_bytes": 0, "d2h_bytes": 0}

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
        so = self.scheduler.schedule()
        self.stats["preemptions"] += len(so.preempted)
        if so.empty:
            return []
        portions, owners = self._portions(so)
        producing = [s for s, p in zip(owners, portions) if p.want]
        ids, logits = self._forward_and_sample(portions, producing, decode_only=not so.prefill)
        st = self.stats
        st["steps"] += 1
        st["tokens"] += so.num_tokens
        st["decode_steps" if not so.prefill else "prefill_steps" if not so.decode else "mixed_steps"] += 1
        outs = []
        for i, seq in enumerate(producing):
            if seq.status != SeqStatus.RUNNING:
                continue
            if seq.params.on_device:
                tok = int(ids[i])
            else:
                row = logits[i].detach().to("cpu", torch.float32).numpy()
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

    def _forward_and_sample(self, portions, producing, decode_only: bool):
        runner, ops = self.runner, self.ops
        R = len(producing)
        for i, seq in enumerate(producing):
            p = seq.params
            device_row = p.on_device and not p.greedy
            self._temp_h[i] = p.temperature if device_row else 0.0
            self._unif_h[i] = seq.sampler.next_uniform() if device_row else 0.0
        # all rows greedy: the row-split argmax kernel picks the tokens; else the sampling kernel (argmax for its greedy rows)
        self._greedy_step = all(s.params.greedy or not s.params.on_device for s in producing)
        bucket = next((b for b in self._buckets if b >= len(portions)), None) if decode_only and self.cuda_graphs else None
        pad = bucket or 0
        starts = runner.prepare(portions, pad_rows=pad, pad_wanted=pad)
        if bucket is not None:
            # a captured step must cover every context it may be replayed with (its launch sizes are fixed)
            runner.meta.max_context = self.max_model_len
        n_w = runner.meta.n_wanted
        if n_w:
            self._temp_h[R:n_w] = 0.0
            self._temp_d[:n_w].copy_(self._temp_h[:n_w], non_blocking=True)
            self._unif_d[:n_w].copy_(self._unif_h[:n_w], non_blocking=True)
        self.stats["h2d_bytes"] += runner.meta.size * 4 + n_w * 12
        logits = None
        if bucket is not None:
            key = (bucket, self._greedy_step)
            g = self._graphs.get(key)
            if g is None:
                logits = self._eager(n_w)              # warm-up: builds, sets kernel attributes, sizes the buffers
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                before = ops.launches
                with torch.cuda.graph(g):
                    self._eager(n_w)
                self.launches_per_graph[key] = ops.launches - before
                self._graphs[key] = g
            g.replay()
            ops.launches += self.launches_per_graph[key]
            self.stats["graph_replays"] += 1
            logits = runner.ws.get("logits", (n_w, self.model.spec.vocab_size), torch.float32)
        else:
            logits = self._eager(n_w)
        runner.commit(portions, starts)
        for p, s in zip(portions, starts):
            self.seqs[p.req].num_computed = s + len(p.tokens)
        ids = None
        if n_w:
            self._ids_h[:n_w].copy_(self._ids_d[:n_w], non_blocking=True)
        ops.errors_to_host()
        if self.model.device.type == "cuda":
            torch.cuda.current_stream(self.model.device).synchronize()
        if n_w:
            ids = self._ids_h[:n_w].numpy()
        self.stats["d2h_bytes"] += n_w * 4 + 4
        ops.check_errors(copied=True)
        return ids, logits

    def _eager(self, n_wanted: int) -> torch.Tensor:
        logits = self.runner.forward()
        if n_wanted and self._greedy_step:
            self.ops.argmax(logits, self._ids_d[:n_wanted])
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
