"""The reference arm of bench.py: the unmodified fusezap package, through its own public API, on the same workload.

The reference is pure Python (its one dependency is numpy; its CUDA backend drives NVRTC and the driver API through
cuda-bindings), so "installing" it is having its `fusezap/` folder under `baseline/_ref/`. Nothing of this repository's
engine, model or kernels is on this path: the model comes from the reference's own random-weights builder
(fusezap/serve/models/random_weights.py:62-72), the steps from its stock engine (fusezap/serve/engine.py:367-369,
542-553, 568-661) with the options `fusezap serve` would give it.

Workload (the same as the other arm's): `batch` requests of seeded uniform token ids whose contexts end at `context`
tokens; after every request decodes, `warmup` untimed steps, then `steps` calls of `engine.step()` timed end to end
by the wall clock with a device synchronisation on both sides (the reference copies ids in and out itself, so there
is no device-only number for it: `value` and `e2e.value` are the same measurement). Then one prompt of
`prefill_tokens` tokens, timed the same way.

Any exception the reference raises ends the arm with `{"impl": "reference", "unavailable": <its text>}`.
"""
from __future__ import annotations
import os
import sys
import tempfile
import time
import traceback

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def shapes_from_config(cfg: dict) -> dict:
    """The reference's shape dictionary (random_weights.py:18-26) from a config.json dictionary."""
    hd = cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]
    if hd != 128:
        raise ValueError(f"the reference's random-weights builder fixes head_dim at 128 (random_weights.py:44); this config has {hd}")
    return dict(hidden_size=cfg["hidden_size"], intermediate_size=cfg["intermediate_size"], n_layers=cfg["num_hidden_layers"],
                n_heads=cfg["num_attention_heads"], n_kv_heads=cfg["num_key_value_heads"], vocab_size=cfg["vocab_size"],
                bias=cfg.get("model_type") == "qwen2", rope_theta=float(cfg.get("rope_theta", 1e4)))


def _say(msg: str) -> None:
    print(f"bench (reference): {msg}", file=sys.stderr, flush=True)


def run(cfg: dict, batch: int, context: int, steps: int, warmup: int, page_size: int, prefill_tokens: int,
        device: str = "CUDA", seed: int = 3, dtype: str = "bfloat16") -> dict:
    """Runs the workload on the reference and returns the measurements; raises what the reference raises."""
    if not os.path.isdir(os.path.join(REF, "fusezap")):
        raise FileNotFoundError("baseline/_ref/fusezap is missing: copy the reference's fusezap/ folder there (it is pure Python)")
    os.environ.setdefault("FZ_CACHE_DIR", os.path.join(tempfile.gettempdir(), f"fusezap-ref-cache-{os.getuid()}"))
    sys.path.insert(0, REF)
    import numpy as np
    from fusezap.dtype import dtypes
    from fusezap.device import Device
    from fusezap.serve.engine import LLMEngine, SamplingParams
    from fusezap.serve.models import random_weights

    sh = shapes_from_config(cfg)
    V = sh["vocab_size"]
    t0 = time.time()
    model = random_weights.build(sh, device, getattr(dtypes, dtype), max_len=context)
    _say(f"model built in {time.time() - t0:.0f}s ({sh['n_layers']} layers)")
    pages = batch * (-(-context // page_size)) + 8
    t0 = time.time()
    eng = LLMEngine(model, num_blocks=pages, block_size=page_size, max_num_seqs=batch, max_model_len=context)
    _say(f"engine ready in {time.time() - t0:.0f}s; prefill sizes {list(eng.prefill_sizes)}, decode sizes {list(eng.decode_sizes)}, "
         f"lookahead {eng.lookahead}")
    dev = Device[model.device]
    rng = np.random.default_rng(seed)
    total = warmup + steps
    n_prompt = context - total - 2
    params = SamplingParams(max_tokens=total + 2, ignore_eos=True)
    rids = [eng.add_request([int(t) for t in rng.integers(0, V, n_prompt)], params) for _ in range(batch)]
    t0 = time.time()
    n_steps = 0
    while any(len(eng.seqs[r].output) == 0 for r in rids):
        eng.step()
        n_steps += 1
        if n_steps > 64 * batch + 64:
            raise RuntimeError("the reference engine did not finish the prompts")
    _say(f"prompts of {n_prompt} tokens done in {time.time() - t0:.0f}s ({n_steps} steps)")
    for _ in range(warmup):
        eng.step()
    dev.synchronize()
    ctx0 = len(eng.seqs[rids[0]].prompt) + len(eng.seqs[rids[0]].output)
    t = time.perf_counter()
    n_tok = 0
    for _ in range(steps):
        n_tok += sum(len(o.new_token_ids) for o in eng.step())
    dev.synchronize()
    dt = time.perf_counter() - t
    out = {"tok_s": n_tok / dt, "ms": dt * 1000.0 / steps, "tokens": n_tok, "context": ctx0 + steps / 2,
           "stats": {k: int(v) for k, v in eng.stats.items() if isinstance(v, (int, float))}}
    for r in rids:
        eng.abort(r)
        eng.release(r)
    # one prompt of prefill_tokens tokens: median of three after a first (compiling) run
    if prefill_tokens and prefill_tokens + 1 <= context:
        ids = [int(x) for x in rng.integers(0, V, prefill_tokens)]
        times = []
        for i in range(4):
            rid = eng.add_request(ids, SamplingParams(max_tokens=1, ignore_eos=True))
            dev.synchronize()
            t = time.perf_counter()
            while eng.has_unfinished():
                eng.step()
            dev.synchronize()
            times.append((time.perf_counter() - t) * 1000.0)
            eng.release(rid)
        ms = sorted(times[1:])[1]
        out["prefill"] = {"value": round(prefill_tokens * 1000.0 / ms, 1), "tokens": prefill_tokens, "ms": round(ms, 3)}
    return out


def unavailable(exc: BaseException) -> str:
    """One line that quotes the exception and where in the reference it was raised."""
    tb = traceback.extract_tb(exc.__traceback__)
    where = next((f"{os.path.relpath(f.filename, REF)}:{f.lineno}" for f in reversed(tb) if f.filename.startswith(REF)), "")
    text = " ".join(str(exc).split())
    if len(text) > 400:
        text = text[:400] + " ..."
    return f"the reference raised {type(exc).__name__}{' at ' + where if where else ''}: {text}"
