"""The engine's host-side logic on the CPU: the package's step function, cache manager, scheduler and entry point run
with the plain kernel table (`plain_ops.PlainOps`) in place of the CUDA one, and are compared with `plain_model`."""
import numpy as np
import pytest
import torch

import plain_model
from fusezap_core_b200 import LLMEngine, SamplingParams, load_model
from fusezap_core_b200.cache import CacheManager, OutOfPages
from fusezap_core_b200.engine import Portion, StepRunner
from plain_ops import PlainOps
from util import lookahead_scenario, make_model_dir, prompts, random_traffic, read_weights


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name in ("tiny_llama", "tiny_qwen2", "tiny_window"):
        d, cfg, opts = make_model_dir(name, tmp_path_factory.mktemp(name))
        out[name] = (load_model(d, "float32", "cpu", max_len=160, ops=PlainOps()), cfg, opts, read_weights(d))
    return out


def runner_for(model, opts, pages, max_len=160):
    cache = CacheManager(model.cache_needs(), model.state_needs(), opts["page_size"], pages, 8, max_len, torch.float32, "cpu")
    return StepRunner(model, cache, max_rows=max_len), cache


@pytest.mark.parametrize("name", ["tiny_llama", "tiny_qwen2", "tiny_window"])
def test_mixed_steps_with_page_reuse_equal_whole_sequences(models, name):
    model, cfg, opts, w = models[name]
    P = prompts(cfg, (37, 22, 51, 9, 30), seed=4)
    ref = [plain_model.forward(cfg, w, ids).numpy() for ids in P]
    pages = 2 * -(-64 // opts["page_size"])          # room for about two requests: pages must be used again
    run, cache = runner_for(model, opts, pages)
    rng = np.random.default_rng(0)
    at = {i: 0 for i in range(len(P))}
    live, waiting, got = [], list(range(len(P))), {i: {} for i in range(len(P))}
    used_pages = set()
    while live or waiting:
        while waiting and len(live) < 3 and cache.can_ensure(("r", waiting[0]), len(P[waiting[0]])) and \
                sum(-(-len(P[i]) // opts["page_size"]) for i in live + [waiting[0]]) <= pages:
            live.append(waiting.pop(0))
        portions = []
        for i in live:
            n = int(min(rng.choice((1, 2, 3, 7, 16)), len(P[i]) - at[i]))
            portions.append((i, Portion(("r", i), P[i][at[i]:at[i] + n], list(range(n)))))
        lg = run.run([p for _, p in portions]).numpy().copy()
        k = 0
        for i, p in portions:
            for j in range(len(p.tokens)):
                got[i][at[i] + j] = lg[k]; k += 1
            at[i] += len(p.tokens)
            used_pages.update(x for x in cache.table(0, ("r", i)) if x >= 0)
            if at[i] == len(P[i]):
                cache.free(("r", i)); live.remove(i)
        cache.check()
    for i in range(len(P)):
        g = np.stack([got[i][p] for p in range(len(P[i]))])
        np.testing.assert_allclose(g, ref[i], rtol=1e-4, atol=2e-5, err_msg=f"request {i}")
    assert cache.num_free_pages == pages


def test_step_refusals(models):
    model, cfg, opts, _ = models["tiny_llama"]
    run, cache = runner_for(model, opts, pages=4, max_len=160)
    with pytest.raises(OutOfPages):
        run.run([Portion("a", list(range(17)), [16])])
    assert cache.num_free_pages == 4
    with pytest.raises(ValueError, match="twice"):
        run.run([Portion("a", [1, 2], []), Portion("a", [3], [0])])
    with pytest.raises(ValueError, match="outside its"):
        run.run([Portion("b", [1, 2], [2])])
    with pytest.raises(ValueError, match="no tokens"):
        run.run([Portion("c", [], [])])
    with pytest.raises(ValueError, match="embedding table"):
        run.run([Portion("d", [cfg["vocab_size"]], [0])])


def greedy_reference(cfg, w, prompt, n):
    ids, out = list(prompt), []
    for _ in range(n):
        t = int(plain_model.forward(cfg, w, ids)[-1].argmax())
        out.append(t); ids.append(t)
    return out


@pytest.mark.parametrize("name,lens,new,chunk", [("tiny_llama", (5, 11, 17), 8, 64), ("tiny_qwen2", (1, 7, 23, 40), 12, 8)])
def test_greedy_generation_through_the_entry_point(models, name, lens, new, chunk):
    model, cfg, opts, w = models[name]
    P = prompts(cfg, lens, seed=1 if name == "tiny_llama" else 2)
    ref = [greedy_reference(cfg, w, p, new) for p in P]
    eng = LLMEngine(model, num_blocks=64, block_size=opts["page_size"], max_num_seqs=4, max_prefill_tokens=chunk, max_model_len=128)
    assert eng.generate(P, SamplingParams(max_tokens=new, ignore_eos=True)) == ref
    if chunk == 8:
        assert eng.stats["mixed_steps"] > 0, "portions of 8 tokens ran beside decoded tokens"
    # so few pages that requests lose them and are recomputed: the same tokens
    few = LLMEngine(model, num_blocks=-(-(max(lens) + new) // opts["page_size"]), block_size=opts["page_size"],
                    max_num_seqs=4, max_prefill_tokens=chunk, max_model_len=128)
    assert few.generate(P, SamplingParams(max_tokens=new, ignore_eos=True)) == ref
    assert few.stats["preemptions"] > 0 and few.cache.num_free_pages == few.cache.num_pages


def test_seeded_sampling_does_not_depend_on_the_batch(models):
    model, cfg, opts, w = models["tiny_qwen2"]
    P = prompts(cfg, (1, 7, 23, 40), seed=2)
    ps = [SamplingParams(max_tokens=12, temperature=0.8, seed=10 + i, ignore_eos=True) for i in range(4)]
    ps[2] = SamplingParams(max_tokens=12, temperature=0.8, top_k=20, top_p=0.9, repetition_penalty=1.2, seed=5, ignore_eos=True)
    ps[3] = SamplingParams(max_tokens=12, temperature=1.3, top_k=12, top_p=0.8, seed=6, ignore_eos=True)   # filters in the kernel table
    mk = lambda: LLMEngine(model, num_blocks=64, block_size=8, max_num_seqs=4, max_prefill_tokens=8, max_model_len=128)
    together = mk().generate(P, ps)
    alone = [mk().generate([p], [q])[0] for p, q in zip(P, ps)]
    assert together == alone
    assert len({tuple(t) for t in together}) == 4 and together != mk().generate(P, SamplingParams(max_tokens=12, ignore_eos=True))
    rng, ids, out = np.random.default_rng(6), list(P[3]), []
    for _ in range(12):
        t = plain_model.sample(plain_model.forward(cfg, w, ids)[-1].numpy(), ids, float(np.float32(1.3)), 12, float(np.float32(0.8)), 1.0, rng)
        out.append(t); ids.append(t)
    assert out == together[3]
    # the sampled tokens follow the plain sampler fed with the plain model's logits
    rng, ids, out = np.random.default_rng(5), list(P[2]), []
    for _ in range(12):
        lg = plain_model.forward(cfg, w, ids)[-1].numpy()
        t = plain_model.sample(lg, ids, 0.8, 20, 0.9, 1.2, rng)
        out.append(t); ids.append(t)
    assert out == together[2]


def test_stop_tokens_abort_and_limits(models):
    model, cfg, opts, w = models["tiny_llama"]
    P = prompts(cfg, (6,), seed=8)
    ref = greedy_reference(cfg, w, P[0], 10)
    eng = LLMEngine(model, num_blocks=32, block_size=4, max_num_seqs=2, max_model_len=64)
    stop = ref[3]
    first = ref.index(stop)
    rid = eng.add_request(P[0], SamplingParams(max_tokens=10, stop_token_ids=[stop]))
    outs = []
    while eng.has_unfinished():
        outs += eng.step()
    assert outs[-1].finished and outs[-1].finish_reason == "stop" and outs[-1].token_ids == ref[:first + 1], "the stop token stays"
    assert outs[-1].num_prompt_tokens == 6 and [o.new_token_ids for o in outs] == [[t] for t in ref[:first + 1]]
    rid = eng.add_request(P[0], SamplingParams(max_tokens=10))
    eng.step(); eng.step()
    o = eng.abort(rid)
    assert o.finished and o.finish_reason == "abort" and not eng.has_unfinished() and eng.cache.num_free_pages == 32
    assert eng.abort(rid) is None
    with pytest.raises(ValueError, match="max_model_len"):
        eng.add_request(list(range(60)), SamplingParams(max_tokens=10))
    with pytest.raises(ValueError, match="vocabulary"):
        eng.add_request([cfg["vocab_size"]], SamplingParams(max_tokens=1))
    eos = LLMEngine(model, num_blocks=32, block_size=4, max_num_seqs=2, max_model_len=64)
    eos.stop_ids = {ref[0]}
    assert eos.generate(P, SamplingParams(max_tokens=10)) == [ref[:1]]
    assert eos.generate(P, SamplingParams(max_tokens=4, ignore_eos=True)) == [ref[:4]]


def test_layer_order_is_data(models, tmp_path):
    """A schedule that names a layer twice (own cache each time) and lets an entry read another entry's cache."""
    import dataclasses
    from fusezap_core_b200.config import ScheduleEntry, describe
    from fusezap_core_b200.engine.model import DecoderModel
    from fusezap_core_b200.weights import load_weights
    d, cfg, opts = make_model_dir("tiny_llama", tmp_path)
    w = read_weights(d)
    typed, spec = describe(cfg)
    spec2 = dataclasses.replace(spec, schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2)))
    m = DecoderModel(spec2, typed)
    ops = PlainOps()
    m.ops = ops
    m.bind(load_weights(d, m.expected_tensors(), "cpu", "float32"), ops, "float32", torch.device("cpu"), 64)
    assert sorted(m.cache_needs()) == [0, 1, 2]
    run, cache = runner_for(m, opts, pages=16, max_len=64)
    ids = prompts(cfg, (21,), seed=6)[0]
    a = run.run([Portion("x", ids[:9], list(range(9)))]).numpy().copy()
    b = run.run([Portion("x", ids[9:], list(range(12)))]).numpy()
    ref = plain_model.forward(cfg, w, ids, schedule=[0, 1, 0]).numpy()
    np.testing.assert_allclose(np.concatenate([a, b]), ref, rtol=1e-4, atol=2e-5)
    # entry 2 runs layer 1's weights again but reads the keys and values entry 1 wrote: it must differ from writing its own
    spec3 = dataclasses.replace(spec, schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(1, 1, write_cache=False)))
    m3 = DecoderModel(spec3, typed); m3.ops = ops
    m3.bind(load_weights(d, m3.expected_tensors(), "cpu", "float32"), ops, "float32", torch.device("cpu"), 64)
    assert sorted(m3.cache_needs()) == [0, 1]
    run3, _ = runner_for(m3, opts, pages=16, max_len=64)
    whole = run3.run([Portion("y", ids, list(range(21)))]).numpy().copy()
    run3.cache.free("y")
    cut = np.concatenate([run3.run([Portion("y", ids[:5], list(range(5)))]).numpy().copy(),
                          run3.run([Portion("y", ids[5:], list(range(16)))]).numpy()])
    np.testing.assert_allclose(cut, whole, rtol=1e-4, atol=2e-5)
    own = plain_model.forward(cfg, w, ids, schedule=[0, 1, 1]).numpy()
    assert np.abs(whole - own).max() > 1e-3


def test_launching_ahead_changes_no_token(models):
    """A decode step launched before the host has read the one before it (its tokens taken from the ids on the device)
    gives the same tokens, ends and reasons as stepping one at a time: through a stop token (the extra token is
    dropped), a length limit (the request is left out), an arrival (looking ahead pauses) and an abort."""
    model, cfg, opts, w = models["tiny_llama"]
    plain, _, _ = lookahead_scenario(model, opts["page_size"], cfg)
    stop = plain[3][12][0]          # request 3's 13th token: it stops there, or earlier if the token comes before
    a, b, eng = lookahead_scenario(model, opts["page_size"], cfg, stop_from=stop)
    assert a == b
    assert eng.stats["lookahead_steps"] > 5
    assert a[3][-1][1:] == (True, "stop") and len(a[3]) <= 13
    assert a[1][-1] == ((), True, "abort") and a[0][-1][1:] == (True, "length") and len(a[2]) == 17


def test_engine_in_one_call(tmp_path):
    """`LLMEngine.from_pretrained` and `from_random` build the model and the engine together."""
    d, cfg, opts = make_model_dir("tiny_llama", tmp_path)
    w = read_weights(d)
    eng = LLMEngine.from_pretrained(d, "float32", "cpu", max_model_len=64, ops=PlainOps(), num_blocks=16, block_size=8,
                                    max_num_seqs=2)
    P = prompts(cfg, (5,), seed=3)
    assert eng.generate(P, SamplingParams(max_tokens=4, ignore_eos=True)) == [greedy_reference(cfg, w, P[0], 4)]
    assert eng.model.generate(P[0], params=SamplingParams(max_tokens=4, ignore_eos=True)) == greedy_reference(cfg, w, P[0], 4)
    rnd = LLMEngine.from_random("tiny-llama", seed=1, dtype="float32", device="cpu", max_model_len=64, ops=PlainOps(),
                                num_blocks=16, block_size=8, max_num_seqs=2)
    assert len(rnd.generate([[1, 2, 3]], SamplingParams(max_tokens=3, ignore_eos=True))[0]) == 3


@pytest.mark.parametrize("seed", [0, 1, 2, 3])
def test_launching_ahead_under_random_traffic(models, seed):
    """Random arrivals, lengths, limits, stop tokens, sampled and greedy requests, aborts and few pages (so that requests
    lose theirs): with and without launching decode steps ahead, every request gets the same tokens and the same end,
    and the cache manager's books are right after every step."""
    model, cfg, opts, w = models["tiny_qwen2"]
    res = random_traffic(model, cfg, seed)
    assert res[False][0] == res[True][0]
    assert res[True][1] > 0 and res[False][1] == 0
    if seed == 0:
        assert res[True][2] > 0 and res[False][2] > 0, "this seed is meant to run out of pages"


@pytest.mark.parametrize("knobs", [dict(prefill_first=2), dict(max_num_batched_tokens=6), dict(mixed_prefill_tokens=3),
                                   dict(prefill_every=2), dict(max_prefill_seqs=1),
                                   dict(prefill_first=1, max_num_batched_tokens=9, max_prefill_seqs=2)])
def test_scheduler_options_change_the_steps_not_the_tokens(models, knobs):
    """Every scheduling option cuts the same work into other steps; each request's tokens stay the same, also with so
    few pages that requests are evicted and recomputed."""
    model, cfg, opts, w = models["tiny_qwen2"]
    P = prompts(cfg, (1, 7, 23, 40), seed=2)
    params = SamplingParams(max_tokens=12, ignore_eos=True)
    base = dict(num_blocks=64, block_size=opts["page_size"], max_num_seqs=4, max_prefill_tokens=8, max_model_len=128)
    plain = LLMEngine(model, **base)
    ref = plain.generate(P, params)
    eng = LLMEngine(model, **base, **knobs)
    assert eng.generate(P, params) == ref
    assert eng.stats["steps"] != plain.stats["steps"] or eng.stats["mixed_steps"] != plain.stats["mixed_steps"]
    if "prefill_first" in knobs:
        assert eng.scheduler.steps_held_back > 0
    few = LLMEngine(model, **dict(base, num_blocks=-(-52 // opts["page_size"]) + 1), **knobs)
    assert few.generate(P, params) == ref and few.stats["preemptions"] > 0 and few.cache.num_free_pages == few.cache.num_pages


def test_engine_takes_one_config_object(models):
    from fusezap_core_b200 import EngineConfig
    model, cfg, opts, w = models["tiny_llama"]
    c = EngineConfig(num_blocks=32, block_size=4, max_num_seqs=3, max_model_len=64, prefill_first=1)
    eng = LLMEngine(model, c)
    assert eng.cfg.max_prefill_tokens == 64 and eng.scheduler.cfg is eng.cfg and eng.cache.page_size == 4
    with pytest.raises(TypeError, match="not both"):
        LLMEngine(model, c, num_blocks=8)
    with pytest.raises(ValueError, match="exceeds the length"):
        LLMEngine(model, max_model_len=100000)
    with pytest.raises(TypeError):
        LLMEngine(model, no_such_option=1)
