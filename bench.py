"""Benchmark: decode tokens per second of the Llama-3.1-8B-sized model (random bf16 weights) on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 4096] [--layers L] [--impl ours|reference]
                    [--preset NAME] [--workload decode|stream]

A "step" is one decode step of `--batch` requests whose contexts end at `--context` tokens. Prints ONE JSON line:
  value      decoded tokens per second, timed on the device (CUDA events around K steps: metadata copy + graph replay)
  e2e        the same through the Python entry point (`LLMEngine.step()`): host token ids in (pinned, copied to the device
             every step), chosen token ids out (copied back every step)
  prefill    one 2,048-token prompt in one step: tokens per second (median of five runs after a warm-up run), and the
             step's FLOPs / time / the measured bf16 peak
  roofline   the decode step's bytes (every weight once + the cache of the live requests) / time, against the measured
             copy bandwidth
  points     decode tokens per second at batch 1 and 64 (contexts ending at `--context`), and at the batch of the main
             run with contexts at the start (prompt length = half of `--context`) and in the middle of generation;
             `points_frac` gives each one's fraction of the copy bandwidth
Peaks come from MEASURED_PEAKS.json beside this file when the driver wrote it, else the fallback figures.
Weights are N(0, 0.02) drawn on the device, prompts are seeded uniform token ids ("data": "synthetic"); the weights
(16 GB) are far larger than the L2, so nothing has to be flushed between steps.

`--workload stream` times a continuous-batching stream instead (by default with the Qwen2.5-0.5B sizes): 32 requests
with prompt lengths uniform in [16, 1024] and 256 new tokens each, one arriving per engine step, through
`LLMEngine.add_request` / `step()`; the line's value is generated tokens per second of wall clock from the first
arrival to the last token.
"""
from __future__ import annotations
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def peaks() -> dict:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown," \
        "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self):
        self.path = os.path.join(tempfile.mkdtemp(), "clocks.csv")
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-f", self.path], stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            with open(self.path) as f:
                for line in f:
                    c = [x.strip() for x in line.split(",")]
                    if len(c) < 8 or not c[0].isdigit():
                        continue
                    sm.append(int(c[0])); mx.append(int(c[1]))
                    for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[4:8]):
                        if v == "Active":
                            reasons.add(name)
        except OSError:
            pass
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def reference_arm(a) -> int:
    """`--impl reference`: the unmodified reference (its `fusezap/` package under baseline/_ref) on the same workload,
    through its own engine; see baseline/reference_arm.py. Prints the same kind of line with "impl": "reference", or
    `{"impl": "reference", "unavailable": why}` when the reference is absent or raises."""
    from baseline import reference_arm as ref
    from fusezap_core_b200.cli import load_preset
    cfg = load_preset(a.preset)
    full_layers = cfg["num_hidden_layers"]
    if a.layers:
        cfg["num_hidden_layers"] = a.layers
    a.warmup = max(a.warmup, 3)
    clocks = ClockSampler()
    clocks.start()
    try:
        r = ref.run(cfg, a.batch, a.context, a.steps, a.warmup, a.page_size, a.prefill_tokens, device=a.reference_device)
    except BaseException as e:      # whatever the reference raises is the record
        clocks.stop()
        if isinstance(e, KeyboardInterrupt):
            raise
        print(json.dumps({"impl": "reference", "unavailable": ref.unavailable(e)}))
        return 0
    clk = clocks.stop()
    Hkv = cfg["num_key_value_heads"]
    hd = cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]
    line = {
        "metric": "decode_tokens_per_s", "value": round(r["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": a.steps,
        "warmup": a.warmup, "ms_per_step": round(r["ms"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "reference",
        "config": {"model": a.preset, "layers": cfg["num_hidden_layers"], "layers_full": full_layers,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": Hkv, "head_dim": hd,
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": a.batch,
                   "seq_len": a.context, "context_mean": round(r["context"], 1), "page_size": a.page_size,
                   "parallelism": "single", "weights": "random N(0,0.02), the reference's own builder",
                   "l2": "inputs larger than L2", "timing": "wall clock around engine.step(), device synchronised"},
        "clocks": clk,
        "e2e": {"value": round(r["tok_s"], 1), "unit": "tok/s", "ms_per_step": round(r["ms"], 4)},
        "prefill": r.get("prefill"),
    }
    print(json.dumps(line))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    ap.add_argument("--preset", default=None,
                    help="layer sizes: llama-3.1-8b (the default of the decode workload), qwen2.5-0.5b (the default of the "
                         "stream workload), qwen2.5-32b, or another preset of the package")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--prefill-prompt", type=int, default=0,
                    help="also time a prompt of this many tokens taken in portions of --prefill-tokens (chunked prefill): "
                         "the whole prompt and its last portion, which has the longest prefix behind it")
    ap.add_argument("--page-size", type=int, default=16, help="tokens per cache page (the engine's block_size)")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 points")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--reference-device", default="CUDA", help="the reference's device name for --impl reference")
    ap.add_argument("--workload", default="decode", choices=["decode", "stream"])
    ap.add_argument("--leave-out", default="", metavar="OPS",
                    help="measurement aid, NOT a benchmark: comma-separated kernel-table operations turned into no-ops "
                         "(e.g. paged_attention, add_rmsnorm, linear_swiglu), to read an operation's cost inside the "
                         "captured step off the difference to a run without it; the line is marked invalid")
    ap.add_argument("--timeline", action="store_true",
                    help="measurement aid: with libraries built with FZB200_NVCC_EXTRA=-DFZ_TIMELINE, print to stderr what "
                         "every kernel of the captured decode step costs on the step's critical path (medians over the "
                         "timed steps); the timestamps cost a little time, so the line is marked invalid")
    ap.add_argument("--no-key-cuts", action="store_true",
                    help="measurement aid: small portions behind long prefixes are not cut along the keys (as before that "
                         "was built); the line says so in `config`")
    ap.add_argument("--requests", type=int, default=32, help="stream workload: number of requests")
    ap.add_argument("--new-tokens", type=int, default=256, help="stream workload: tokens generated per request")
    a = ap.parse_args()
    if a.preset is None and a.workload != "stream":
        a.preset = "llama-3.1-8b"
    if a.impl == "reference":
        return reference_arm(a)
    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    a.warmup = max(a.warmup, 3)
    if a.workload == "stream":
        return stream_workload(a)

    import numpy as np
    import torch
    from fusezap_core_b200 import LLMEngine, SamplingParams
    from fusezap_core_b200.cli import load_preset
    from fusezap_core_b200.engine import Portion
    from fusezap_core_b200.engine.model import random_model

    cfg = load_preset(a.preset)
    full_layers = cfg["num_hidden_layers"]
    if a.layers:
        cfg["num_hidden_layers"] = a.layers
    L = cfg["num_hidden_layers"]
    pk = peaks()
    dev = torch.device("cuda:0")
    page = a.page_size
    t0 = time.time()
    model = random_model(cfg, "bfloat16", dev, seed=0, max_len=a.context)
    torch.cuda.synchronize()
    if a.no_key_cuts:
        model.ops.cut_prefill_keys = False
    left_out = [name for name in a.leave_out.split(",") if name]
    for name in left_out:
        if not callable(getattr(model.ops, name, None)):
            raise SystemExit(f"--leave-out: the kernel table has no operation {name!r}")
        setattr(model.ops, name, lambda *args, **kw: None)      # (a fused operation that returns None falls back to its parts)
    print(f"bench: model built in {time.time() - t0:.1f}s, {model.weight_bytes() / 1e9:.2f} GB of weights read per step",
          file=sys.stderr, flush=True)
    Hkv, hd = cfg["num_key_value_heads"], cfg["head_dim"]
    kv_bytes_per_token = 2 * Hkv * hd * 2 * L
    rng = np.random.default_rng(3)
    V = cfg["vocab_size"]

    def make_engine(batch: int) -> LLMEngine:
        pages = batch * (-(-a.context // page)) + 8
        # prefill_first: while prompts are pending the requests that already decode wait, so all of them start
        # decoding together, at equal contexts
        return LLMEngine(model, num_blocks=pages, block_size=page, max_num_seqs=batch, max_prefill_tokens=a.prefill_tokens,
                         max_model_len=a.context, prefill_first=1 << 30, lookahead=False)

    def prefill_to(eng: LLMEngine, batch: int, n_prompt: int, max_tokens: int) -> list[int]:
        """Admits `batch` requests of n_prompt seeded tokens and steps until every one decodes."""
        rids = [eng.add_request(rng.integers(0, V, n_prompt).tolist(), SamplingParams(max_tokens=max_tokens, ignore_eos=True))
                for _ in range(batch)]
        while any(not eng.requests[r].decoding for r in rids):
            eng.step()
        return rids

    def decode_run(batch: int, steps: int, warmup: int, e2e: bool, ctx_end: int | None = None) -> dict:
        """Times `steps` decode steps of `batch` requests whose contexts end at ctx_end (default a.context)."""
        eng = make_engine(batch)
        total = steps + warmup
        runs = 2 if e2e else 1
        n_prompt = (ctx_end or a.context) - runs * total - 2
        rids = prefill_to(eng, batch, n_prompt, max_tokens=runs * total + 2)
        out = {}
        # device-timed: metadata copy + graph replay per step, tokens fixed beforehand, no read-back inside
        runner, meta = eng.runner, eng.runner.meta
        seqs = [eng.requests[r] for r in rids]
        bucket = next(b for b in eng._buckets if b >= batch)
        def graph_key():      # the captured step of this bucket (greedy rows, ids picked on the device)
            return next(k for k in eng._graphs if k[0] == bucket)
        def one_step(i: int):
            portions = [Portion(s.rid, [s.token(s.cached)], [0]) for s in seqs]
            starts = runner.prepare(portions, pad_rows=bucket, pad_wanted=bucket)
            eng._graphs[graph_key()].replay()
            runner.commit(portions, starts)
            for s, st in zip(seqs, starts):   # the next token is fixed beforehand: nothing is read back in this loop
                s.cached = st + 1
                s.generated.append(int((s.rid * 7919 + i) % V))
        eng.step()                      # builds the graph of this bucket
        for i in range(warmup - 1):
            one_step(i)
        torch.cuda.synchronize()
        launches0 = model.ops.launches
        ctx0 = seqs[0].cached
        if a.timeline:
            from fusezap_core_b200.kernels import timeline
            timeline.read(model.ops)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(steps):
            one_step(i)
        end.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(end) / steps
        if a.timeline:
            events = timeline.read(model.ops)
            per = len(events) // steps
            rows = timeline.per_launch_costs(events[: per * steps], per)
            print(f"timeline: batch {batch}, {steps} steps of {per} launches; per launch in step order: source file, cost on "
                  f"the critical path, first block resident before its dependency was met", file=sys.stderr)
            for i, r in enumerate(rows):
                print(f"  {i:4d} {r['file']:16s} {r['cost_us']:8.2f} us {r['resident_before_us']:8.2f} us", file=sys.stderr)
        ctx_mean = ctx0 + steps / 2
        out.update(ms=ms, tok_s=batch * 1000.0 / ms, context=ctx_mean,
                   launches=steps * eng.launches_per_graph.get(graph_key(), 0) + (model.ops.launches - launches0),
                   bytes=model.weight_bytes() + batch * ctx_mean * kv_bytes_per_token)
        if e2e:
            eng.lookahead = True        # the entry point's default; off above, where the steps are driven by hand
            for _ in range(warmup):
                eng.step()
            torch.cuda.synchronize()
            h0, d0 = eng.stats["h2d_bytes"], eng.stats["d2h_bytes"]
            t = time.perf_counter()
            n_tok = 0
            for _ in range(steps):
                n_tok += len(eng.step())
            torch.cuda.synchronize()
            dt = time.perf_counter() - t
            out.update(e2e_tok_s=n_tok / dt, e2e_ms=dt * 1000 / steps, h2d=(eng.stats["h2d_bytes"] - h0) // steps,
                       d2h=(eng.stats["d2h_bytes"] - d0) // steps)
        for r in rids:
            eng.abort(r)
        del eng
        torch.cuda.empty_cache()
        return out

    def prefill_run(tokens: int) -> dict:
        eng = make_engine(1)
        ids = rng.integers(0, V, tokens).tolist()
        times = []
        for i in range(6):      # one warm-up, then the median of five
            rid = eng.add_request(ids, SamplingParams(max_tokens=1, ignore_eos=True))
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            eng.step()
            end.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(end))
            eng.release(rid)
        ms = sorted(times[1:])[2]
        D, I, Hq = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_attention_heads"]
        lin = 2 * tokens * L * (D * (Hq + 2 * Hkv) * hd + Hq * hd * D + 3 * D * I) + 2 * D * V
        attn = 2 * tokens * tokens * hd * Hq * L     # causal: half of 4 T^2 hd Hq
        flops = lin + attn
        return {"value": round(tokens * 1000.0 / ms, 1), "tokens": tokens, "ms": round(ms, 3),
                "frac": round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4), "flops": flops}

    def chunked_prefill_run(prompt: int, portion: int) -> dict:
        """A prompt longer than a step's portion: one engine step per portion, each timed; median of three prompts."""
        eng = make_engine(1)
        ids = rng.integers(0, V, prompt).tolist()
        totals, lasts = [], []
        for i in range(4):      # one warm-up prompt (it also records the by-shape graphs), then three timed ones
            rid = eng.add_request(ids, SamplingParams(max_tokens=1, ignore_eos=True))
            per_step = []
            while not eng.requests[rid].generated:
                torch.cuda.synchronize()
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                eng.step()
                end.record()
                torch.cuda.synchronize()
                per_step.append(start.elapsed_time(end))
            eng.release(rid)
            totals.append(sum(per_step))
            lasts.append(per_step[-1])
        total, last = sorted(totals[1:])[1], sorted(lasts[1:])[1]
        return {"prompt": prompt, "portion": portion, "portions": len(per_step), "ms_total": round(total, 3),
                "value": round(prompt * 1000.0 / total, 1), "ms_last_portion": round(last, 3),
                "last_portion_tokens": prompt - (len(per_step) - 1) * portion}

    clocks = ClockSampler()
    clocks.start()
    main_run = decode_run(a.batch, a.steps, a.warmup, e2e=not a.no_e2e)
    clk = clocks.stop()
    pre = prefill_run(a.prefill_tokens)
    chunked = chunked_prefill_run(a.prefill_prompt, a.prefill_tokens) if a.prefill_prompt > a.prefill_tokens else None
    points, points_frac = {}, {}
    if not a.no_points:
        def point(name: str, batch: int, ctx_end: int | None = None) -> None:
            r = decode_run(batch, max(48, a.steps), max(8, a.warmup), e2e=False, ctx_end=ctx_end)
            points[name] = round(r["tok_s"], 1)
            points_frac[name] = round(r["bytes"] / (r["ms"] * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        point("decode_b1", 1)
        point("decode_b64", 64)
        # the main batch where generation starts (after a prompt of half the context) and half-way through it
        point(f"decode_b{a.batch}_ctx_start", a.batch, a.context // 2 + max(48, a.steps) + max(8, a.warmup) + 2)
        point(f"decode_b{a.batch}_ctx_mean", a.batch, 3 * a.context // 4)
    achieved = main_run["bytes"] / (main_run["ms"] * 1e-3) / 1e9
    line = {
        "metric": "decode_tokens_per_s", "value": round(main_run["tok_s"], 1), "unit": "tok/s", "n_gpus": 1,
        "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(main_run["ms"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {"model": a.preset, "layers": L, "layers_full": full_layers, "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": Hkv, "head_dim": hd, "intermediate": cfg["intermediate_size"],
                   "vocab": V, "global_batch": a.batch, "seq_len": a.context, "context_mean": round(main_run["context"], 1),
                   "page_size": page, "parallelism": "single", "weights": "random N(0,0.02)", "l2": "inputs larger than L2",
                   "peaks": pk["source"]},
        "clocks": clk,
        "e2e": ({"value": round(main_run["e2e_tok_s"], 1), "unit": "tok/s", "ms_per_step": round(main_run["e2e_ms"], 4),
                 "h2d_bytes_per_step": int(main_run["h2d"]), "d2h_bytes_per_step": int(main_run["d2h"])} if not a.no_e2e else None),
        "gpu_launches": int(main_run["launches"]),
        "prefill": {k: pre[k] for k in ("value", "tokens", "ms", "frac")},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "points_frac": points_frac,
    }
    if chunked is not None:
        line["chunked_prefill"] = chunked
    if a.no_key_cuts:
        line["config"]["key_cuts"] = "off"
    if a.timeline:
        line["invalid"] = "timeline timestamps in every kernel"
    if left_out:
        line["invalid"] = "operations left out: " + ", ".join(left_out)
    print(json.dumps(line))
    return 0


def stream_workload(a) -> int:
    """A continuous-batching stream (see the module docstring). One JSON line."""
    import numpy as np
    import torch
    from fusezap_core_b200 import LLMEngine, SamplingParams
    from fusezap_core_b200.cli import load_preset
    from fusezap_core_b200.engine.model import random_model
    preset = a.preset or "qwen2.5-0.5b"
    cfg = load_preset(preset)
    full_layers = cfg["num_hidden_layers"]
    if a.layers:
        cfg["num_hidden_layers"] = a.layers
    max_len = 1024 + a.new_tokens
    model = random_model(cfg, "bfloat16", "cuda:0", seed=0, max_len=max_len)
    rng = np.random.default_rng(5)
    lens = rng.integers(16, 1025, a.requests)
    prompts = [rng.integers(0, cfg["vocab_size"], int(n)).tolist() for n in lens]
    params = SamplingParams(max_tokens=a.new_tokens, ignore_eos=True)
    pages = a.requests * (-(-max_len // a.page_size)) + 8

    def run_once() -> dict:
        eng = LLMEngine(model, num_blocks=pages, block_size=a.page_size, max_num_seqs=a.requests,
                        max_prefill_tokens=a.prefill_tokens, max_model_len=max_len)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        nxt = n_tok = n_steps = 0
        first = {}
        while nxt < len(prompts) or eng.has_unfinished():
            if nxt < len(prompts):
                eng.add_request(prompts[nxt], params)
                nxt += 1
            for o in eng.step():
                n_tok += len(o.new_token_ids)
                first.setdefault(o.request_id, time.perf_counter() - t0)
            n_steps += 1
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        return {"s": dt, "tok_s": n_tok / dt, "tokens": n_tok, "steps": n_steps, "stats": dict(eng.stats),
                "launches": model.ops.launches}

    run_once()                       # warm-up: builds every graph the stream needs
    clocks = ClockSampler()
    clocks.start()
    launches0 = model.ops.launches
    runs = [run_once() for _ in range(3)]
    clk = clocks.stop()
    r = sorted(runs, key=lambda x: x["s"])[1]
    line = {
        "metric": "stream_generated_tokens_per_s", "value": round(r["tok_s"], 1), "unit": "tok/s", "n_gpus": 1,
        "steps": r["steps"], "warmup": 1, "ms_per_step": round(1000 * r["s"] / r["steps"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {"model": preset, "layers": cfg["num_hidden_layers"], "layers_full": full_layers,
                   "requests": a.requests, "prompt_len_min": 16, "prompt_len_max": 1024, "new_tokens": a.new_tokens,
                   "prompt_tokens": int(lens.sum()), "arrivals": "one per engine step", "page_size": a.page_size,
                   "max_prefill_tokens": a.prefill_tokens, "timing": "wall clock, median of 3 runs after one warm-up run"},
        "clocks": clk,
        "e2e": {"value": round(r["tok_s"], 1), "unit": "tok/s", "seconds": round(r["s"], 4),
                "prompt_tokens_per_s": round(float(lens.sum()) / r["s"], 1)},
        "gpu_launches": int((model.ops.launches - launches0) // 3),
        "engine_stats": {k: r["stats"][k] for k in ("steps", "decode_steps", "prefill_steps", "mixed_steps", "graph_replays",
                                                      "step_graph_replays", "lookahead_steps", "preemptions")},
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
