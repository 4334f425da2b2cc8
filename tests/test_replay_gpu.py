"""Trace replay on the GPU: the same requests cut in every way give the logits of the plain implementation.

For each tiny configuration and both dtypes one `bin/trace_run` process replays, one after the other:
  whole    each request alone, whole, in one step
  last32   most of a request in one step, its last 32 tokens one by one
  portions portions of changing size, down to two tokens
  mixed    up to four live requests, portions of some beside single tokens of others, in a pool so small that pages
           given back by finished requests are used again by later ones
and every wanted position is compared with `plain_model.forward` of the whole request. In float32 the four cuttings
must also agree with each other bit for bit (the reference asserts the same of its engine:
tests/test_serve_cuda.py:847-866): every sum's order is a function of the row alone.
"""
import numpy as np
import pytest

from util import TraceBuilder, assert_close, make_model_dir, plain_logits, prompts, read_weights, run_trace

pytestmark = pytest.mark.gpu

LENGTHS = (70, 41, 97, 33, 58, 64)   # six requests; the pool below holds the four short ones at a time
POOL_TOKENS = 256


def build_trace(P: list[list[int]]) -> TraceBuilder:
    tb = TraceBuilder()
    # 1. whole: each request alone
    for i, ids in enumerate(P):
        tb.step([(f"w{i}", ids, "all")], end=[f"w{i}"])
    # 2. most of it in one step, the last 32 tokens one by one
    for i, ids in enumerate(P[:3]):
        cut = len(ids) - 32
        tb.step([(f"d{i}", ids[:cut], "all")])
        for t in range(cut, len(ids)):
            tb.step([(f"d{i}", ids[t:t + 1], [0])], end=[f"d{i}"] if t == len(ids) - 1 else [])
    # 3. portions of changing size, down to two tokens
    sizes = (7, 2, 13, 3, 2, 16, 5, 2, 31, 4)
    for i, ids in enumerate(P[:3]):
        at, k = 0, i
        while at < len(ids):
            n = min(sizes[k % len(sizes)], len(ids) - at)
            tb.step([(f"p{i}", ids[at:at + n], "all")], end=[f"p{i}"] if at + n == len(ids) else [])
            at, k = at + n, k + 1
    # 4. mixed: a little scheduler that keeps up to four requests live; a request first gets portions of its prompt
    # part (two thirds), then single tokens; finished requests give their pages back and the next one starts
    rng = np.random.default_rng(5)
    waiting = sorted(range(len(P)), key=lambda i: -(-len(P[i]) // 64))     # the four that fit together come first
    live: dict[int, int] = {}
    held = 0
    budget = POOL_TOKENS   # tokens the pool holds, each request rounded up to 64
    tb.most_live = 0
    while waiting or live:
        while waiting and len(live) < 4 and held + -(-len(P[waiting[0]]) // 64) * 64 <= budget:
            i = waiting.pop(0)
            live[i] = 0
            held += -(-len(P[i]) // 64) * 64
        tb.most_live = max(tb.most_live, len(live))
        entries, ends = [], []
        for i in list(live):
            at, ids = live[i], P[i]
            if rng.random() < 0.2 and len(live) > 1:
                continue   # a request may be left out of a step
            n = 1 if at >= 2 * len(ids) // 3 else int(min(rng.integers(2, 12), len(ids) - at))
            entries.append((f"m{i}", ids[at:at + n], "all"))
            live[i] = at + n
            if live[i] == len(ids):
                ends.append(f"m{i}")
                del live[i]
                held -= -(-len(ids) // 64) * 64
        if entries:
            tb.step(entries, end=ends)
    return tb


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_llama", "tiny_qwen2", "tiny_window", "tiny_hd64", "tiny_hd128"])
def test_replay_all_cuttings(name, dtype, tmp_path):
    model_dir, cfg, opts = make_model_dir(name, tmp_path, "float32")
    weights = read_weights(model_dir)
    P = prompts(cfg, LENGTHS, seed=3)
    ref = [plain_logits(cfg, weights, ids, dtype) for ids in P]
    tb = build_trace(P)
    assert tb.most_live == 4 and max(len(s["entries"]) for s in tb.steps) == 4, "four requests live, and in one step"
    outs = run_trace(model_dir, dtype, str(tmp_path / "out"), max_tokens=POOL_TOKENS, steps=tb.steps, page_size=opts["page_size"])
    got = tb.collect(outs, cfg["vocab_size"])
    for rid, rows in sorted(got.items()):
        i = int(rid[1:])
        assert sorted(rows) == list(range(len(P[i]))), f"{rid}: positions {sorted(rows)[:5]}..."
        g = np.stack([rows[p] for p in range(len(P[i]))])
        assert_close(g, ref[i], dtype, f"{name} {dtype} request {rid}")
    assert {r[0] for r in got} == {"w", "d", "p", "m"}
    if dtype == "float32":
        # bit for bit among the cuttings: whole / last 32 one by one / portions / mixed
        for rid, rows in sorted(got.items()):
            if rid[0] == "w":
                continue
            whole = got["w" + rid[1:]]
            for p, row in rows.items():
                assert np.array_equal(row, whole[p]), (f"{name}: request {rid} position {p} differs from the whole request's "
                                                       f"row by {np.abs(row - whole[p]).max():.3e}")


def test_replay_default_pages_bf16_file(tmp_path):
    """A bfloat16 checkpoint, the default page size (16), float32 and bfloat16 compute."""
    model_dir, cfg, _ = make_model_dir("tiny_qwen2", tmp_path, "bfloat16")
    weights = read_weights(model_dir)
    P = prompts(cfg, (50, 19), seed=9)
    for dtype in ("float32", "bfloat16"):
        tb = TraceBuilder()
        tb.step([("a", P[0][:30], [29]), ("b", P[1], "all")])
        tb.step([("a", P[0][30:], "all")], end=["a", "b"])
        outs = run_trace(model_dir, dtype, str(tmp_path / f"out-{dtype}"), max_tokens=128, steps=tb.steps)
        got = tb.collect(outs, cfg["vocab_size"])
        ref = [plain_logits(cfg, weights, ids, dtype) for ids in P]
        g = np.stack([got["a"][p] for p in sorted(got["a"])])
        assert sorted(got["a"]) == list(range(29, 50))
        assert_close(g, ref[0][29:], dtype, f"a {dtype}")
        assert_close(np.stack([got["b"][p] for p in range(19)]), ref[1], dtype, f"b {dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page", [("tiny_hd128", 64), ("tiny_hd64", 16)])
def test_replay_beyond_4096_positions(name, page, dtype, tmp_path):
    """A 4,400-token request: portions of 1,500, then the last 32 tokens one by one, beside a short second request. Past
    key 4096 the decode kernel cuts the key axis in larger units, the prompt kernel walks 35 key tiles, and pages of 64 are
    fetched as one TMA box."""
    model_dir, cfg, opts = make_model_dir(name, tmp_path, "float32")
    weights = read_weights(model_dir)
    P = prompts(cfg, (4400, 70), seed=5)
    ref = [plain_logits(cfg, weights, ids, dtype) for ids in P]
    tb = TraceBuilder()
    long_ids, short = P
    at = 0
    for n in (1500, 1500, 1368):
        tb.step([("L", long_ids[at:at + n], [n - 1])])
        at += n
    tb.step([("L", long_ids[at:at + 1], [0]), ("S", short[:60], [59])])
    at += 1
    k = 60
    while at < len(long_ids):
        entries = [("L", long_ids[at:at + 1], [0])]
        if k < len(short):
            entries.append(("S", short[k:k + 2], "all")); k += 2
        tb.step(entries, end=(["S"] if k >= len(short) and len(entries) == 2 else []))
        at += 1
    outs = run_trace(model_dir, dtype, str(tmp_path / "out"), max_tokens=4608, steps=tb.steps, page_size=page, timeout=900)
    got = tb.collect(outs, cfg["vocab_size"])
    for rid, i in (("L", 0), ("S", 1)):
        pos = sorted(got[rid])
        g = np.stack([got[rid][p] for p in pos])
        assert_close(g, ref[i][pos], dtype, f"{name} {dtype} request {rid}")
    assert max(got["L"]) == 4399 and len(got["L"]) >= 35
