"""The engine on the GPU through the Python entry point and the command line: greedy generation, long decoding, the
first tokens of a sequence, sampling, CUDA graphs on and off, few pages."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_model
from util import ROOT, STD_SCALE, lookahead_scenario, make_model_dir, plain_logits, prompts, random_traffic, read_weights

pytestmark = pytest.mark.gpu


def follows_plain_model(cfg, w, dtype, prompt, toks, margin):
    """Every generated token is the plain model's argmax, or within `margin` of it (a near tie)."""
    wr = w if dtype == "float32" else {k: v.to(torch.bfloat16) for k, v in w.items()}
    act = torch.float32 if dtype == "float32" else torch.bfloat16
    lg = plain_model.forward(cfg, wr, list(prompt) + list(toks), act).numpy()
    for i, t in enumerate(toks):
        row = lg[len(prompt) - 1 + i]
        assert row.max() - row[t] <= margin, f"{dtype}: token {i} = {t} has logit {row[t]:.4f}, the maximum is {row.max():.4f}"


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {n: make_model_dir(n, tmp_path_factory.mktemp(n)) for n in ("tiny_llama", "tiny_qwen2", "tiny_window", "tiny_hd64",
                                                                        "tiny_hd128")}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,lens,new,chunk", [("tiny_llama", (5, 11, 17), 8, 64), ("tiny_qwen2", (1, 7, 23, 40), 12, 8),
                                                 ("tiny_window", (3, 30, 14), 20, 8)])
def test_greedy_generation(folders, name, lens, new, chunk, dtype):
    from fusezap_core_b200 import LLMEngine, SamplingParams, load_model
    d, cfg, opts = folders[name]
    w = read_weights(d)
    P = prompts(cfg, lens, seed=1 if name == "tiny_llama" else 2)
    model = load_model(d, dtype, "cuda:0", max_len=128)
    margin = 1e-3 if dtype == "float32" else 0.15
    outs = {}
    for graphs in (True, False):
        eng = LLMEngine(model, num_blocks=64, block_size=opts["page_size"], max_num_seqs=4, max_prefill_tokens=chunk,
                        max_model_len=128, cuda_graphs=graphs)
        outs[graphs] = eng.generate(P, SamplingParams(max_tokens=new, ignore_eos=True))
        assert (eng.stats["graph_replays"] > 0) == graphs
        assert eng.cache.num_free_pages == 64
    assert outs[True] == outs[False], "replaying captured steps changes no token"
    for p, t in zip(P, outs[True]):
        assert len(t) == new
        follows_plain_model(cfg, w, dtype, p, t, margin)
    # so few pages that requests lose theirs and are recomputed
    few = LLMEngine(model, num_blocks=-(-(max(lens) + new) // opts["page_size"]), block_size=opts["page_size"],
                    max_num_seqs=4, max_prefill_tokens=chunk, max_model_len=128)
    again = few.generate(P, SamplingParams(max_tokens=new, ignore_eos=True))
    assert few.stats["preemptions"] > 0
    if dtype == "float32":
        assert again == outs[True], "float32: a row's bits do not depend on the batch or the cut, so neither do the tokens"
    for p, t in zip(P, again):
        follows_plain_model(cfg, w, dtype, p, t, margin)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(folders, dtype):
    """200 tokens decoded one by one from a one-token prompt: the first tokens of a sequence (positions 0, 1, 2, ...),
    every page boundary, and a context of hundreds of keys."""
    from fusezap_core_b200 import LLMEngine, SamplingParams, load_model
    d, cfg, opts = folders["tiny_qwen2"]
    w = read_weights(d)
    model = load_model(d, dtype, "cuda:0", max_len=256)
    eng = LLMEngine(model, num_blocks=40, block_size=8, max_num_seqs=2, max_model_len=256)
    toks = eng.generate([[17]], SamplingParams(max_tokens=200, ignore_eos=True))[0]
    assert len(toks) == 200
    follows_plain_model(cfg, w, dtype, [17], toks, 1e-3 if dtype == "float32" else 0.15)


@pytest.mark.parametrize("dtype,graphs", [("float32", True), ("float32", False), ("bfloat16", True)])
def test_launching_ahead_changes_no_token(folders, dtype, graphs):
    """Decode steps launched before the host has read the step before (their tokens taken from the ids on the device)
    give the same tokens, ends and reasons as one step at a time, through a stop token, length limits, a late arrival
    and an abort. In bfloat16 without the stop token: a request that runs one token too many would change the batch
    size of that step, and with it the rounding of the others."""
    from fusezap_core_b200 import load_model
    d, cfg, opts = folders["tiny_llama"]
    model = load_model(d, dtype, "cuda:0", max_len=128)
    stop = None
    if dtype == "float32":
        plain, _, _ = lookahead_scenario(model, opts["page_size"], cfg, graphs)
        stop = plain[3][12][0]
    a, b, eng = lookahead_scenario(model, opts["page_size"], cfg, graphs, stop_from=stop)
    assert a == b
    assert eng.stats["lookahead_steps"] > 5
    if stop is not None:
        assert a[3][-1][1:] == (True, "stop")
    assert a[1][-1] == ((), True, "abort") and a[0][-1][1:] == (True, "length") and len(a[2]) == 17


@pytest.mark.parametrize("seed,graphs", [(0, True), (5, True), (6, False)])
def test_launching_ahead_under_random_traffic(folders, seed, graphs):
    """The random story of `util.random_traffic` on the GPU in float32 (a row's bits do not depend on the batch, so the
    tokens must be equal): tokens fed on the device, captured steps, requests that lose their pages."""
    from fusezap_core_b200 import load_model
    d, cfg, opts = folders["tiny_qwen2"]
    model = load_model(d, "float32", "cuda:0", max_len=128)
    res = random_traffic(model, cfg, seed, graphs)
    assert res[False][0] == res[True][0]
    assert res[True][1] > 0 and res[False][1] == 0


def test_small_steps_replay_captured_graphs(folders):
    """Portions of 8 prompt tokens with decoded tokens of other requests beside them: the second step of a shape is
    captured and later ones replay it. In float32 a row's bits do not depend on the batch, so the tokens must be those
    of an engine that launches every kernel itself."""
    from fusezap_core_b200 import LLMEngine, SamplingParams, load_model
    d, cfg, opts = folders["tiny_qwen2"]
    model = load_model(d, "float32", "cuda:0", max_len=128)
    P = prompts(cfg, (41, 33, 38, 29, 44, 35), seed=4)
    ps = [SamplingParams(max_tokens=9 + i, ignore_eos=True) for i in range(len(P))]
    ps[1] = SamplingParams(max_tokens=10, temperature=0.9, top_k=15, top_p=0.85, seed=3, ignore_eos=True)
    mk = lambda graphs: LLMEngine(model, num_blocks=96, block_size=8, max_num_seqs=4, max_prefill_tokens=8,
                                  max_model_len=128, cuda_graphs=graphs)
    with_graphs, without = mk(True), mk(False)
    assert with_graphs.generate(P, ps) == without.generate(P, ps)
    assert with_graphs.stats["step_graph_replays"] > 4 and without.stats["graph_replays"] == 0
    assert with_graphs.cache.num_free_pages == with_graphs.cache.num_pages
    # an engine told not to capture such steps replays decode steps only
    only_decode = LLMEngine(model, num_blocks=96, block_size=8, max_num_seqs=4, max_prefill_tokens=8, max_model_len=128, graph_rows=0)
    assert only_decode.generate(P, ps) == without.generate(P, ps) and only_decode.stats["step_graph_replays"] == 0


@pytest.mark.parametrize("name", ["tiny_hd64", "tiny_hd128"])
def test_the_serving_path_at_tensor_core_head_sizes(folders, name):
    """bfloat16 at head sizes 64 and 128, where attention runs on the tensor-core kernels (portions of 8 tokens and more
    on the tcgen05 kernel, decoded tokens on the split-key kernel): the composition that serving and the benchmark use,
    through the scheduler, with decode steps replayed from per-bucket graphs whose launch sizes cover `max_model_len`
    (much larger than any live context here), mixed steps replayed from by-shape graphs, and decode steps launched
    ahead. Contexts cross a 64-key unit and a 256-key block of the split-key kernel while decoding. The few-token kernels
    compute a row independently of the other rows of a step and of padding, so graphs on / off and launching ahead on /
    off must give equal tokens, not merely close ones; and the tokens follow the plain bfloat16 model."""
    from fusezap_core_b200 import LLMEngine, SamplingParams, load_model
    d, cfg, opts = folders[name]
    w = read_weights(d)
    model = load_model(d, "bfloat16", "cuda:0", max_len=1024)
    P = prompts(cfg, (250, 60, 5, 130, 33, 71), seed=9)
    ps = [SamplingParams(max_tokens=n, ignore_eos=True) for n in (14, 12, 20, 9, 16, 11)]
    outs, engines = {}, {}
    for graphs in (True, False):
        for ahead in (True, False):
            eng = LLMEngine(model, num_blocks=80, block_size=16, max_num_seqs=4, max_prefill_tokens=48, max_model_len=1024,
                            cuda_graphs=graphs, lookahead=ahead)
            seen = {}
            launch = eng._launch
            def spy(portions, rows, decode_only, all_produce, kind="decode_steps", eng=eng, seen=seen, launch=launch):
                out = launch(portions, rows, decode_only, all_produce, kind)
                m = eng.runner.meta
                # (the plan tells the decode attention kernel when every portion is a single token)
                assert m.plan.single_tokens == all(len(p.tokens) == 1 for p in portions)
                assert m.plan.single_tokens or not decode_only
                if not decode_only:
                    sig = (m.n_rows, m.n_wanted, *eng.ops.step_signature(m))
                    seen.setdefault(sig, set()).add(tuple((sg.row0, sg.n, sg.pos0) for sg in m.segments))
                return out
            eng._launch = spy
            outs[graphs, ahead] = eng.generate(P, ps)
            engines[graphs, ahead] = (eng, seen)
            model.ops.check_errors()
            assert eng.cache.num_free_pages == 80
    eng, seen = engines[True, True]
    assert eng.stats["graph_replays"] > 10 and eng.stats["step_graph_replays"] > 0 and eng.stats["lookahead_steps"] > 5
    assert any(len(layouts) > 1 and sig[2] > 0 for sig, layouts in seen.items()), \
        "two steps with equal sizes but different portion layouts, with rows on the tile kernel"
    assert engines[False, False][0].stats["graph_replays"] == 0 and engines[False, False][0].stats["lookahead_steps"] == 0
    for k, v in outs.items():
        assert v == outs[False, False], f"graphs {k[0]}, launching ahead {k[1]}: tokens differ from kernel-by-kernel stepping"
    for p, t, q in zip(P, outs[True, True], ps):
        assert len(t) == q.max_tokens
        follows_plain_model(cfg, w, "bfloat16", p, t, 0.15)
    # so few pages that requests lose theirs and are recomputed (as portions, on the other attention kernel: close, not equal)
    few = LLMEngine(model, num_blocks=-(-270 // 16) + 3, block_size=16, max_num_seqs=4, max_prefill_tokens=48, max_model_len=1024)
    again = few.generate(P, ps)
    assert few.stats["preemptions"] > 0 and few.cache.num_free_pages == few.cache.num_pages
    for p, t in zip(P, again):
        follows_plain_model(cfg, w, "bfloat16", p, t, 0.15)


def test_small_portions_of_a_long_prompt(tmp_path):
    """A prompt of 2,500 tokens run in portions of 160 behind one another (head size 128, bfloat16): from 2,048 cached
    keys on, the one or two query tiles of a portion are cut along the keys into pieces that a second kernel merges,
    inside steps that are replayed from by-shape graphs. The tokens that follow the prompt are those of the plain model,
    with the cuts and with the cuts switched off."""
    import copy
    from fusezap_core_b200 import LLMEngine, SamplingParams, load_model
    from fusezap_core_b200.weights import write_random_model
    from tiny_configs import get
    cfg, opts = get("tiny_hd128")
    cfg = copy.deepcopy(cfg)
    cfg["max_position_embeddings"] = 4096
    d = str(tmp_path / "tiny_hd128_long")
    write_random_model(cfg, d, opts["seed"], "float32", opts["norm_noise"], std_scale=STD_SCALE)
    w = read_weights(d)
    model = load_model(d, "bfloat16", "cuda:0", max_len=4096)
    P = prompts(cfg, (2500,), seed=4)
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    outs, plans = {}, {}
    try:
        for cut in (True, False):
            model.ops.cut_prefill_keys = cut
            eng = LLMEngine(model, num_blocks=200, block_size=16, max_num_seqs=2, max_prefill_tokens=160, max_model_len=4096)
            seen = []
            launch = eng._launch
            def spy(portions, rows, decode_only, all_produce, kind="decode_steps", eng=eng, seen=seen, launch=launch):
                out = launch(portions, rows, decode_only, all_produce, kind)
                plan = eng.runner.meta.plan
                seen.append((plan.n_tiles, plan.n_cuts, plan.n_pieces))
                return out
            eng._launch = spy
            outs[cut] = eng.generate(P, sp)
            plans[cut] = seen
            model.ops.check_errors()
            assert eng.stats["step_graph_replays"] > 0, "portions of equal shape replay a captured step"
    finally:
        model.ops.cut_prefill_keys = True
    assert sum(1 for _, c, _ in plans[True] if c > 0) >= 2 and max(p for _, _, p in plans[True]) >= 4
    assert all(c == 0 for _, c, _ in plans[False])
    for toks in outs.values():
        follows_plain_model(cfg, w, "bfloat16", P[0], toks[0], 0.15)


@pytest.mark.parametrize("dtype,name", [("float32", "tiny_qwen2"), ("bfloat16", "tiny_hd128")])
def test_scheduler_options_through_the_engine(folders, dtype, name):
    """`prefill_first`, `max_num_batched_tokens` (also below `max_num_seqs`, where the decode buckets must not outgrow
    a step), `mixed_prefill_tokens`, `prefill_every`, `max_prefill_seqs`: other steps, and in float32 the same tokens
    as the default engine (a row's bits do not depend on the batch or the cut); in bfloat16 tokens that follow the
    plain model."""
    from fusezap_core_b200 import LLMEngine, SamplingParams, load_model
    d, cfg, opts = folders[name]
    w = read_weights(d)
    model = load_model(d, dtype, "cuda:0", max_len=256)
    P = prompts(cfg, (30, 7, 55, 12, 41, 3, 26, 18), seed=5)
    params = SamplingParams(max_tokens=10, ignore_eos=True)
    base = dict(num_blocks=96, block_size=opts["page_size"], max_num_seqs=8, max_prefill_tokens=16, max_model_len=256)
    ref = LLMEngine(model, **base).generate(P, params)
    for knobs in (dict(prefill_first=2), dict(max_num_batched_tokens=20), dict(max_num_batched_tokens=6),
                  dict(mixed_prefill_tokens=5, prefill_every=2), dict(max_prefill_seqs=1, prefill_first=1)):
        eng = LLMEngine(model, **base, **knobs)
        got = eng.generate(P, params)
        model.ops.check_errors()
        assert eng.stats["graph_replays"] > 0 and eng.cache.num_free_pages == 96
        if "prefill_first" in knobs:
            assert eng.scheduler.steps_held_back > 0
        if knobs.get("max_num_batched_tokens") == 6:
            assert max(eng._buckets) == 6, "no decode bucket is larger than a step may be"
        if dtype == "float32":
            assert got == ref, knobs
        else:
            for p, t in zip(P, got):
                follows_plain_model(cfg, w, dtype, p, t, 0.15)


def test_seeded_sampling_on_the_device(folders):
    from fusezap_core_b200 import LLMEngine, SamplingParams, load_model
    d, cfg, opts = folders["tiny_qwen2"]
    w = read_weights(d)
    P = prompts(cfg, (1, 7, 23, 40), seed=2)
    model = load_model(d, "float32", "cuda:0", max_len=128)
    ps = [SamplingParams(max_tokens=12, temperature=0.8, seed=10 + i, ignore_eos=True) for i in range(4)]
    ps[2] = SamplingParams(max_tokens=12, temperature=0.8, top_k=20, top_p=0.9, repetition_penalty=1.2, seed=5, ignore_eos=True)
    ps[3] = SamplingParams(max_tokens=12, temperature=1.3, top_k=12, top_p=0.8, seed=6, ignore_eos=True)   # filters on the device
    mk = lambda: LLMEngine(model, num_blocks=64, block_size=8, max_num_seqs=4, max_prefill_tokens=8, max_model_len=128)
    together = mk().generate(P, ps)
    alone = [mk().generate([p], [q])[0] for p, q in zip(P, ps)]
    assert together == alone, "a request's draws do not depend on the batch"
    # request 3 (top-k and top-p, picked on the device): every token lies in the set the plain filters keep
    ids = list(P[3])
    for t in together[3]:
        lg = plain_model.forward(cfg, w, ids)[-1].numpy().astype(np.float64) / float(np.float32(1.3))
        kept = plain_model.top_p_filter(plain_model.top_k_filter(lg, 12), float(np.float32(0.8)))
        assert np.isfinite(kept[t]) and np.isfinite(kept).sum() <= 12
        ids.append(t)
    # request 0 (temperature only, picked on the device) against the plain sampler on the plain model's logits
    rng, ids = np.random.default_rng(10), list(P[0])
    for t in together[0]:
        lg = plain_model.forward(cfg, w, ids)[-1].numpy().astype(np.float64) / 0.8
        e = np.exp(lg - lg.max()); c = np.cumsum(e); u = rng.random() * c[-1]
        want = int(np.searchsorted(c, u, side="right"))
        near = abs(c[want] - u) < 1e-4 * c[-1] or (want > 0 and abs(c[want - 1] - u) < 1e-4 * c[-1])
        assert t == want or near
        ids.append(t)


def test_command_line(folders, tmp_path):
    d, cfg, opts = folders["tiny_llama"]
    cmd = [sys.executable, "-m", "fusezap_core_b200", "generate", d, "--dtype", "float32", "--prompt-ids", "5,17,3,200",
           "--prompt-lens", "9", "--prompt-seed", "4", "--max-tokens", "5", "--ignore-eos", "--max-model-len", "64",
           "--num-blocks", "32", "--block-size", "4", "--max-num-seqs", "2"]
    p = subprocess.run(cmd, capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [json.loads(l) for l in p.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 2 and all(len(l["token_ids"]) == 5 and l["finish_reason"] == "length" for l in lines)
    assert lines[0]["num_prompt_tokens"] == 4 and lines[1]["num_prompt_tokens"] == 9
    w = read_weights(d)
    follows_plain_model(cfg, w, "float32", [5, 17, 3, 200], lines[0]["token_ids"], 1e-3)
    # the scheduler's options on the command line: other steps, the same tokens (float32); and the per-step profile
    p2 = subprocess.run(cmd + ["--prefill-first", "2", "--max-num-batched-tokens", "5", "--max-prefill-tokens", "4",
                               "--mixed-prefill-tokens", "3", "--profile"], capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert p2.returncode == 0, p2.stderr[-2000:]
    assert [json.loads(l)["token_ids"] for l in p2.stdout.splitlines() if l.startswith("{")] == [l["token_ids"] for l in lines]
    assert "profile:" in p2.stderr and "paged_attention" in p2.stderr and "linear" in p2.stderr
    out = str(tmp_path / "rw")
    p = subprocess.run([sys.executable, "-m", "fusezap_core_b200", "random-weights", "--preset", "tiny-qwen2", "--out", out,
                        "--seed", "3", "--dtype", "bfloat16"], capture_output=True, text=True, cwd=ROOT, timeout=120)
    assert p.returncode == 0 and os.path.isfile(os.path.join(out, "model.safetensors")) and os.path.isfile(os.path.join(out, "config.json"))
    # a preset with random weights instead of a folder; the same seed gives the same tokens, and the replay subcommand runs
    runs = []
    for _ in range(2):
        p = subprocess.run([sys.executable, "-m", "fusezap_core_b200", "generate", "--random", "tiny-qwen2", "--random-seed", "5",
                            "--prompt-ids", "1,2,3", "--max-tokens", "4", "--ignore-eos", "--max-model-len", "64",
                            "--num-blocks", "16", "--max-num-seqs", "2"], capture_output=True, text=True, cwd=ROOT, timeout=300)
        assert p.returncode == 0, p.stderr[-2000:]
        runs.append([json.loads(l)["token_ids"] for l in p.stdout.splitlines() if l.startswith("{")])
    assert runs[0] == runs[1] and len(runs[0][0]) == 4
    p = subprocess.run([sys.executable, "-m", "fusezap_core_b200", "replay", "--model", out, "--dtype", "bfloat16", "--out",
                        str(tmp_path / "lg"), "--max-tokens", "64"], input='{"step": 0, "entries": [{"id": "a", "tokens": [5, 6, 7], "want": [2]}], "end": ["a"]}\n',
                       capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert p.returncode == 0 and "done 0" in p.stdout and os.path.getsize(str(tmp_path / "lg" / "0.f32")) == 4 * 384, p.stderr[-2000:]


def test_no_gpu_tensor_no_run(folders):
    from fusezap_core_b200.kernels import cuda_ops
    from fusezap_core_b200.kernels.table import KernelError
    with pytest.raises(KernelError, match="CUDA device only"):
        cuda_ops("float32", "cpu")
