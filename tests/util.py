"""Helpers shared by the tests: tiny model folders in temporary directories, plain reference logits, tolerances."""
from __future__ import annotations
import json
import os
import subprocess
import sys

import numpy as np
import torch

import plain_model
from tiny_configs import get

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
STD_SCALE = 4.0   # N(0, 0.08) instead of N(0, 0.02): tiny models with the smaller weights give near-constant logits


def make_model_dir(name: str, tmp: str, dtype: str = "float32") -> tuple[str, dict, dict]:
    """Writes the tiny configuration `name` with seeded random weights; returns (folder, config.json dict, options)."""
    from fusezap_core_b200.weights import write_random_model
    cfg, opts = get(name)
    d = os.path.join(str(tmp), f"{name}-{dtype}")
    write_random_model(cfg, d, opts["seed"], dtype, opts["norm_noise"], std_scale=STD_SCALE)
    return d, cfg, opts


def read_weights(model_dir: str) -> dict[str, torch.Tensor]:
    """Checkpoint tensors through the `safetensors` package (not through the package under test)."""
    from safetensors.torch import load_file
    return load_file(os.path.join(model_dir, "model.safetensors"))


def plain_logits(cfg: dict, weights: dict, ids, dtype: str) -> np.ndarray:
    """Reference logits (T, V) of one whole request. bfloat16: weights and stored activations rounded to bfloat16."""
    if dtype == "bfloat16":
        w = {k: v.to(torch.bfloat16) for k, v in weights.items()}
        return plain_model.forward(cfg, w, ids, torch.bfloat16).numpy()
    return plain_model.forward(cfg, weights, ids, torch.float32).numpy()


def tolerance(dtype: str, ref: np.ndarray, longest_sum: int = 256) -> tuple[float, float]:
    """(atol, rtol) for single logits. float32: the reduction class of the reference's tests (tests/conftest.py:20-24
    there: 1e-4, 1e-5), a little tighter in atol, for sums of up to 256 terms (the tiny models). The engine's float32
    products are one fmaf chain over k, whose rounding error grows like sqrt(k) against a blocked CPU sum, so for
    longer sums (`longest_sum`: the largest k of any product, e.g. 14336 at Llama-3.1-8B sizes) atol grows by
    sqrt(longest_sum / 256). bfloat16: eight bfloat16 steps (2^-8 each) at the scale of the largest
    logit: rounding the stored activations to bfloat16 moves the plain implementation's own logits by up to four such
    steps on these models (measured: 0.008 to 0.015 of the scale), and two roundings of that size differ by more."""
    if dtype == "float32":
        return 2e-5 * max(1.0, (longest_sum / 256.0) ** 0.5), 1e-4
    return float(np.abs(ref).max()) * 2.0 ** -5, 0.0


def assert_close(got: np.ndarray, ref: np.ndarray, dtype: str, what: str = "", longest_sum: int = 256) -> None:
    """Every logit within `tolerance`, and in bfloat16 every row's root-mean-square difference within two bfloat16
    steps of the scale (rounding alone gives 0.002 to 0.003 of the scale; a wrong key, page or position gives far more)."""
    atol, rtol = tolerance(dtype, ref, longest_sum)
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    err = np.abs(got - ref) - (atol + rtol * np.abs(ref))
    if dtype != "float32" and got.ndim == 2:
        rms = np.sqrt(((got - ref) ** 2).mean(axis=-1))
        lim = float(np.abs(ref).max()) * 2.0 ** -7
        bad = np.where(rms > lim)[0]
        assert len(bad) == 0, (f"{what}: rows {bad[:8].tolist()} differ by rms {rms[bad[0]]:.3e} > {lim:.3e}; "
                               f"first wrong row {bad[0]} of {got.shape[0]}, {len(bad)} wrong rows")
    if err.max() > 0:
        i = np.unravel_index(np.argmax(err), err.shape)
        rows = np.where((err > 0).any(axis=-1))[0] if err.ndim == 2 else []
        raise AssertionError(f"{what}: max |diff| {np.abs(got - ref).max():.3e} (atol {atol:.2e}, rtol {rtol:.0e}) at {i}: "
                             f"got {got[i]:.6f}, expected {ref[i]:.6f}; first wrong row {rows[0] if len(rows) else '-'} "
                             f"of {got.shape[0]}, {len(rows)} wrong rows")


def prompts(cfg: dict, lengths, seed: int) -> list[list[int]]:
    rng = np.random.default_rng(seed)
    return [rng.integers(0, cfg["vocab_size"], n).tolist() for n in lengths]


# ---------------------------------------------------------------- trace replay
def run_trace(model_dir: str, dtype: str, out_dir: str, max_tokens: int, steps: list[dict], page_size: int | None = None,
              timeout: int = 600) -> dict[int, np.ndarray]:
    """Runs bin/trace_run on `steps`; returns {step: raw float32 array} for the steps that wrote logits."""
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype, "--out", out_dir,
           "--max-tokens", str(max_tokens)]
    if page_size:
        cmd += ["--page-size", str(page_size)]
    text = "".join(json.dumps(s) + "\n" for s in steps)
    p = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=timeout)
    assert p.returncode == 0, f"trace_run exit {p.returncode}\nstdout:\n{p.stdout[-2000:]}\nstderr:\n{p.stderr[-4000:]}"
    done = [l for l in p.stdout.splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == [s["step"] for s in steps], "trace_run did not acknowledge every step"
    out = {}
    for s in steps:
        fn = os.path.join(out_dir, f"{s['step']}.f32")
        if os.path.exists(fn):
            out[s["step"]] = np.fromfile(fn, dtype="<f4")
    return out


class TraceBuilder:
    """Builds trace steps and remembers which (request, position) each wanted row is."""
    def __init__(self):
        self.steps: list[dict] = []
        self.where: dict[int, list[tuple[str, int]]] = {}
        self.fed: dict[str, int] = {}

    def step(self, entries: list[tuple[str, list[int], list[int] | str]], end: list[str] = ()) -> None:
        """entries: (request id, tokens, want) with want a list of places or "all"."""
        n = len(self.steps)
        es, where = [], []
        for rid, toks, want in entries:
            want = list(range(len(toks))) if want == "all" else list(want)
            base = self.fed.get(rid, 0)
            es.append({"id": rid, "tokens": [int(t) for t in toks], "want": want})
            where += [(rid, base + j) for j in want]
            self.fed[rid] = base + len(toks)
        self.steps.append({"step": n, "entries": es, "end": list(end)})
        self.where[n] = where
        for rid in end:
            self.fed.pop(rid, None)

    def collect(self, outs: dict[int, np.ndarray], vocab: int) -> dict[str, dict[int, np.ndarray]]:
        """{request: {position: logits row}} from the files trace_run wrote."""
        got: dict[str, dict[int, np.ndarray]] = {}
        for n, where in self.where.items():
            if not where:
                assert n not in outs, f"step {n} wrote logits nobody wanted"
                continue
            a = outs[n].reshape(len(where), vocab)
            for (rid, p), row in zip(where, a):
                got.setdefault(rid, {})[p] = row
        return got


def lookahead_scenario(model, page_size, cfg, graphs=True, stop_from=None):
    """Runs one fixed story (different lengths, a stop token, a device-sampled request, a late arrival, an abort) with
    and without launching steps ahead and returns both per-request records and the engine that looked ahead."""
    from fusezap_core_b200 import LLMEngine, SamplingParams
    P = prompts(cfg, (5, 11, 3, 8, 6), seed=21)
    res = {}
    for ahead in (False, True):
        eng = LLMEngine(model, num_blocks=96, block_size=page_size, max_num_seqs=4, max_prefill_tokens=16,
                        max_model_len=96, cuda_graphs=graphs, lookahead=ahead)
        ps = [SamplingParams(max_tokens=3, ignore_eos=True), SamplingParams(max_tokens=25, ignore_eos=True),
              SamplingParams(max_tokens=17, temperature=0.7, seed=3, ignore_eos=True),
              SamplingParams(max_tokens=30, ignore_eos=True, stop_token_ids=list(stop_from or ())),
              SamplingParams(max_tokens=9, ignore_eos=True)]
        rids = [eng.add_request(P[i], ps[i]) for i in range(4)]
        rec = {r: [] for r in rids}
        n = 0
        while eng.has_unfinished():
            for o in eng.step():
                rec[o.request_id].append((tuple(o.new_token_ids), o.finished, o.finish_reason))
            n += 1
            if n == 7:
                r = eng.add_request(P[4], ps[4]); rec[r] = []; rids.append(r)
            if n == 15:
                o = eng.abort(rids[1])
                rec[rids[1]].append(((), o.finished, o.finish_reason))
        assert eng.cache.num_free_pages == 96
        eng.cache.check()
        res[ahead] = (rec, eng)
    return res[False][0], res[True][0], res[True][1]


def random_traffic(model, cfg, seed, graphs=True):
    """Runs one random story of requests (arrivals, lengths, limits, stop tokens, sampled and greedy ones, an abort, few
    pages) with and without launching decode steps ahead. Returns {ahead: (records per request, steps launched ahead,
    preemptions)}; the cache manager's books are checked after every step."""
    from fusezap_core_b200 import LLMEngine, SamplingParams
    rng = np.random.default_rng(seed)
    n_req = 9
    lens = rng.integers(1, 40, n_req)
    P = prompts(cfg, tuple(int(x) for x in lens), seed=100 + seed)
    arrive = np.sort(rng.integers(0, 25, n_req))
    params = []
    for i in range(n_req):
        kind = rng.integers(0, 3)
        params.append(SamplingParams(max_tokens=int(rng.integers(1, 30)), ignore_eos=True,
                                     temperature=0.8 if kind == 1 else 0.0, seed=int(rng.integers(0, 1000)),
                                     top_k=5 if kind == 2 and rng.random() < 0.5 else 0,
                                     stop_token_ids=[int(t) for t in rng.integers(0, cfg["vocab_size"], 12)]))
    abort_at = {int(rng.integers(5, 40)): int(rng.integers(0, n_req))}
    res = {}
    for ahead in (False, True):
        eng = LLMEngine(model, num_blocks=14, block_size=8, max_num_seqs=4, max_prefill_tokens=16, max_model_len=96,
                        lookahead=ahead, cuda_graphs=graphs)
        rec, rids, step, nxt = {}, {}, 0, 0
        while nxt < n_req or eng.has_unfinished():
            while nxt < n_req and arrive[nxt] <= step:
                rids[nxt] = eng.add_request(P[nxt], params[nxt]); rec[rids[nxt]] = []; nxt += 1
            for o in eng.step():
                rec[o.request_id].append((tuple(o.new_token_ids), o.finished, o.finish_reason))
            eng.cache.check()
            step += 1
            if step in abort_at and abort_at[step] in rids:
                o = eng.abort(rids[abort_at[step]])
                if o is not None:
                    rec[o.request_id].append(((), True, "abort"))
            assert step < 2000
        assert eng.cache.num_free_pages == 14
        res[ahead] = (rec, eng.stats["lookahead_steps"], eng.stats["preemptions"])
    return res
