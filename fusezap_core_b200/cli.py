"""Command line: `python -m fusezap_core_b200 <command>`.

  generate MODEL          run prompts (token ids) through the engine and print each request's new tokens as JSON
  random-weights          write a model folder (config.json, model.safetensors) from a configuration and a seed
  build                   compile the CUDA kernels now

Engine options carry the names, meanings and defaults of the reference's `fusezap serve`
(fusezap/serve/cli.py:8-41): --dtype auto|float32|bfloat16 (auto: bfloat16), --max-model-len 2048, --max-num-seqs 32,
--max-prefill-tokens, --num-blocks 1024, --block-size 16, --device, and the scheduler's own (--max-num-batched-tokens,
--max-prefill-seqs, --mixed-prefill-tokens, --prefill-every, --prefill-first); they are generated from `EngineConfig`,
which holds their defaults. Sampling options are those of the reference's `SamplingParams`
(fusezap/serve/engine.py:39-50). The reference's text side (tokenizer, HTTP) is not part of this engine: prompts are
token ids.
"""
from __future__ import annotations
import argparse
import json
import os
import sys
import time

PRESET_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "config", "presets")


def presets() -> list[str]:
    return sorted(f[:-5] for f in os.listdir(PRESET_DIR) if f.endswith(".json"))


def load_preset(name: str) -> dict:
    path = os.path.join(PRESET_DIR, name + ".json")
    if not os.path.isfile(path):
        raise SystemExit(f"unknown preset {name!r} (have {presets()})")
    with open(path) as f:
        return json.load(f)


def add_engine_options(s: argparse.ArgumentParser) -> None:
    """The engine's options: one flag per field of `EngineConfig`, which also holds their defaults and meanings."""
    from .config import EngineConfig
    EngineConfig.add_arguments(s)


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="fusezap_core_b200", description="B200-native engine for the dense Llama / Qwen2.5 decoder")
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("generate", help="generate tokens for prompts given as token ids")
    g.add_argument("model", nargs="?", default=None, help="model folder (config.json + safetensors)")
    g.add_argument("--random", default=None, metavar="PRESET",
                   help=f"instead of a model folder: the sizes of a preset ({', '.join(presets())}) with random weights")
    g.add_argument("--random-seed", type=int, default=0, help="seed of the random weights")
    add_engine_options(g)
    g.add_argument("--prompt-ids", action="append", default=[], help="comma-separated token ids; repeat for more prompts")
    g.add_argument("--prompt-file", default=None, help="JSON lines, each a list of token ids")
    g.add_argument("--prompt-lens", default=None, help="comma-separated lengths of random prompts (with --prompt-seed)")
    g.add_argument("--prompt-seed", type=int, default=0)
    g.add_argument("--max-tokens", type=int, default=16)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-k", type=int, default=0)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--repetition-penalty", type=float, default=1.0)
    g.add_argument("--seed", type=int, default=None, help="sampling seed; request i uses seed + i")
    g.add_argument("--stop-token-ids", default="", help="comma-separated")
    g.add_argument("--ignore-eos", action="store_true")
    r = sub.add_parser("random-weights", help="write a model folder with seeded random weights")
    r.add_argument("--preset", default=None, help=f"one of {presets()}")
    r.add_argument("--config", default=None, help="a config.json to take the sizes from")
    r.add_argument("--out", required=True)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--dtype", default="bfloat16", choices=["float32", "bfloat16"])
    r.add_argument("--norm-noise", action="store_true", help="norm weights 1 + N(0, 0.02) instead of 1")
    r.add_argument("--num-layers", type=int, default=None, help="override the layer count")
    sub.add_parser("build", help="compile the CUDA kernels")
    sub.add_parser("replay", add_help=False, help="trace replay: token ids from standard input, logits to files "
                                                   "(the options of bin/trace_run)")
    sub.add_parser("bench", add_help=False, help="the benchmark of the source tree (bench.py beside the package)")
    return ap


def build_engine(a: argparse.Namespace):
    from .config import EngineConfig
    from .engine.llm_engine import LLMEngine
    if (a.model is None) == (a.random is None):
        raise SystemExit("give a model folder or --random PRESET (one of them)")
    cfg = EngineConfig.from_arguments(a)
    if a.random is not None:
        eng = LLMEngine.from_random(load_preset(a.random), seed=a.random_seed, config=cfg)
        a.model = f"random {a.random} (seed {a.random_seed})"
    else:
        eng = LLMEngine.from_pretrained(a.model, config=cfg)
    return eng


def cmd_generate(a: argparse.Namespace) -> int:
    import numpy as np
    from .sampling import SamplingParams
    t0 = time.perf_counter()
    eng = build_engine(a)
    print(f"fusezap_core_b200: loaded {a.model} on {eng.cfg.device} ({eng.cfg.dtype}) in {time.perf_counter() - t0:.1f}s",
          file=sys.stderr, flush=True)
    prompts = [[int(t) for t in p.split(",") if t.strip()] for p in a.prompt_ids]
    if a.prompt_file:
        with open(a.prompt_file) as f:
            prompts += [json.loads(line) for line in f if line.strip()]
    if a.prompt_lens:
        rng = np.random.default_rng(a.prompt_seed)
        V = eng.model.spec.vocab_size
        prompts += [rng.integers(0, V, int(n)).tolist() for n in a.prompt_lens.split(",")]
    if not prompts:
        raise SystemExit("no prompts: give --prompt-ids, --prompt-file or --prompt-lens")
    stop = [int(t) for t in a.stop_token_ids.split(",") if t.strip()]
    params = [SamplingParams(max_tokens=a.max_tokens, temperature=a.temperature, top_k=a.top_k, top_p=a.top_p,
                             repetition_penalty=a.repetition_penalty, seed=None if a.seed is None else a.seed + i,
                             stop_token_ids=stop, ignore_eos=a.ignore_eos) for i in range(len(prompts))]
    t0 = time.perf_counter()
    rids = [eng.add_request(p, q) for p, q in zip(prompts, params)]
    done = {}
    while eng.has_unfinished():
        for out in eng.step():
            if out.finished:
                done[out.request_id] = out
    dt = time.perf_counter() - t0
    for rid in rids:
        o = done[rid]
        print(json.dumps({"request_id": rid, "num_prompt_tokens": o.num_prompt_tokens, "token_ids": o.token_ids,
                          "finish_reason": o.finish_reason}))
    n = sum(len(done[r].token_ids) for r in rids)
    print(f"fusezap_core_b200: {n} tokens in {dt:.2f}s ({n / dt:.1f} tok/s), {eng.stats}", file=sys.stderr, flush=True)
    if eng.profile:
        from .kernels.profile import format_report
        print(format_report(eng.profile_report()), file=sys.stderr, flush=True)
    return 0


def cmd_random_weights(a: argparse.Namespace) -> int:
    from .weights import write_random_model
    if bool(a.preset) == bool(a.config):
        raise SystemExit("give exactly one of --preset and --config")
    if a.preset:
        cfg = load_preset(a.preset)
    else:
        with open(a.config) as f:
            cfg = json.load(f)
    if a.num_layers:
        cfg["num_hidden_layers"] = a.num_layers
    write_random_model(cfg, a.out, a.seed, a.dtype, a.norm_noise)
    print(f"fusezap_core_b200: wrote {a.out} (seed {a.seed}, {a.dtype})", file=sys.stderr)
    return 0


def main(argv: list[str] | None = None) -> int:
    argv = sys.argv[1:] if argv is None else list(argv)
    if argv and argv[0] == "replay":          # its options are its own: hand the rest over
        from .replay import main as replay_main
        return replay_main(argv[1:])
    if argv and argv[0] == "bench":
        import runpy
        path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py")
        if not os.path.exists(path):
            raise SystemExit(f"bench.py is not beside the package (looked for {path})")
        sys.argv = [path] + argv[1:]
        runpy.run_path(path, run_name="__main__")
        return 0
    a = build_parser().parse_args(argv)
    if a.cmd == "generate":
        return cmd_generate(a)
    if a.cmd == "random-weights":
        return cmd_random_weights(a)
    if a.cmd == "build":
        from .kernels.build import build_all
        for so in build_all():
            print(so)
        return 0
    return 2
