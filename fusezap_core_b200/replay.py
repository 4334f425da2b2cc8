"""Trace replay: feeds given token ids through a model step by step and writes the logits. It samples nothing.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N [--page-size P]
    python -m fusezap_core_b200 replay --model DIR ...            (the same)

Steps come on standard input, one JSON object a line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
All entries of a step run as one batch through the engine's own step function, cache manager and kernels: this module
has no forward pass, cache or loader of its own. For a step that wants logits, `DIR/<step>.f32` receives them as
little-endian float32 [wanted, vocab], in the order of the entries and of `want`. After every step a line `done <step>`
is printed and flushed. `end` lists requests whose pages are given back after the step. The pool holds --max-tokens
tokens (in pages of --page-size, default 16), so pages are reused.
"""
import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True, help="most tokens live requests hold at any time")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--device", default="cuda:0")
    a = ap.parse_args(argv)

    import numpy as np
    import torch
    from .cache import CacheManager
    from .engine import Portion, StepRunner, load_model

    os.makedirs(a.out, exist_ok=True)
    ps = a.page_size
    num_pages = -(-a.max_tokens // ps)
    max_len = num_pages * ps
    model = load_model(a.model, a.dtype, a.device, max_len=max_len)
    cache = CacheManager(model.cache_needs(), model.state_needs(), ps, num_pages, max_requests=64,
                         max_model_len=max_len, dtype=model.ops.dtype, device=model.device)
    runner = StepRunner(model, cache, max_rows=max_len, max_wanted=max_len, max_segments=64)
    runner.ws.row_capacity = min(max_len, 512)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        portions = [Portion(e["id"], e["tokens"], e.get("want", [])) for e in step.get("entries", [])]
        if portions:
            logits = runner.run(portions)
            if logits.shape[0]:
                out = logits.detach().to("cpu", torch.float32).numpy().astype("<f4", copy=False)
                out.tofile(os.path.join(a.out, f"{step['step']}.f32"))
            model.ops.check_errors()
        for rid in step.get("end", []):
            cache.free(rid)
        print(f"done {step['step']}", flush=True)
    return 0
