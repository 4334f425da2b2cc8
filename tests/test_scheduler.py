"""The scheduler's decisions alone (no model): a fake token function drives it, and after every step the invariants
are checked, in the manner of the reference's tests/test_scheduler.py:26-135."""
import random

import pytest
import torch

from fusezap_core_b200.cache import CacheManager, KVNeed
from fusezap_core_b200.config import EngineConfig
from fusezap_core_b200.engine.request import Phase, Request
from fusezap_core_b200.engine.scheduler import Scheduler


class P:   # what the scheduler needs of sampling params
    def __init__(self, max_tokens): self.max_tokens = max_tokens


def make(pages=16, page_size=4, max_len=64, **cfg):
    cache = CacheManager({0: KVNeed(1, 16, 0)}, {}, page_size, pages, 8, max_len, torch.float32, "cpu", allocate=False)
    return Scheduler(EngineConfig(num_blocks=pages, block_size=page_size, max_model_len=max_len, **cfg), cache), cache


def run(sch, cache, reqs, arrivals=None, max_steps=2000):
    """Drives the scheduler as the engine does. Returns the list of plans."""
    plans, pending = [], sorted(arrivals.items()) if arrivals else []
    step = 0
    cfg = sch.cfg
    while sch.has_unfinished() or pending:
        while pending and pending[0][0] <= step:
            sch.submit(pending.pop(0)[1])
        generating_before = sum(1 for r in sch.live if r.decoding)
        plan = sch.plan()
        step += 1
        assert step < max_steps, "the scheduler does not finish"
        # invariants of one step
        assert len({id(w.request) for w in plan.work}) == len(plan.work), "a request twice in one step"
        assert plan.num_tokens <= cfg.token_budget
        prompt_tokens = sum(n for _, _, n in plan.portions)
        assert prompt_tokens <= cfg.max_prefill_tokens
        assert len(plan.portions) <= (cfg.max_prefill_seqs or cfg.max_num_seqs)
        if plan.decode and cfg.mixed_prefill_tokens:
            assert prompt_tokens <= cfg.mixed_prefill_tokens
        if plan.decode and cfg.prefill_every > 1 and sch.steps % cfg.prefill_every:
            assert prompt_tokens == 0
        assert len(sch.live) <= cfg.max_num_seqs
        assert [r.order for r in sch.live] == sorted(r.order for r in sch.live)
        assert [r.order for r in sch.queue] == sorted(r.order for r in sch.queue)
        if plan.held_back:
            assert not plan.decode and plan.portions and plan.held_back == generating_before
        for v in plan.evicted:
            assert v.cached == 0 and v.phase is Phase.QUEUED and not cache.holds(v.rid)
            assert all(v is not w.request for w in plan.work), "a request that lost its pages runs in the same step"
        for w in plan.work:
            r = w.request
            assert w.start == r.cached and 1 <= w.count <= r.pending and (not w.decode or w.count == 1)
            assert len(cache.table(0, r.rid)) * cache.page_size >= w.start + w.count, "rows without pages"
        cache.check()
        for w in plan.work:
            r = w.request
            r.cached += w.count
            cache.commit(r.rid, r.cached)
            if r.cached == r.known:
                r.generated.append(1000 + len(r.generated))
                if len(r.generated) >= r.params.max_tokens:
                    sch.retire(r, "length")
        plans.append(plan)
    assert cache.num_free_pages == cache.num_pages
    return plans


def req(i, n_prompt, max_tokens, order=None):
    return Request(i, list(range(n_prompt)), P(max_tokens), order=i if order is None else order)


def kinds(plans):
    return "".join("p" if p.portions and not p.decode else "d" if p.decode and not p.portions else "m" if p.work else "-"
                   for p in plans)


def test_prompt_is_cut_into_portions_under_the_budget():
    sch, cache = make(max_num_seqs=4, max_prefill_tokens=8)
    r = req(0, 20, 3)
    sch.submit(r)
    plans = run(sch, cache, [r])
    assert [[n for _, _, n in p.portions] for p in plans[:3]] == [[8], [8], [4]]
    assert [len(p.decode) for p in plans] == [0, 0, 0, 1, 1] and r.ended_by == "length" and len(r.generated) == 3


def test_portions_and_decoded_tokens_share_a_step():
    sch, cache = make(max_num_seqs=4, max_prefill_tokens=8)
    a, b = req(0, 4, 6), req(1, 20, 2)
    sch.submit(a)
    plans = run(sch, cache, [a, b], arrivals={2: b})
    assert kinds(plans).count("m") >= 2, "a prompt portion runs beside a decoded token"


def test_head_of_queue_is_never_skipped():
    sch, cache = make(pages=8, page_size=4, max_len=32, max_num_seqs=4, max_prefill_tokens=64)
    big, small1, small2 = req(0, 24, 4), req(1, 14, 2), req(2, 2, 2)
    for r in (big, small1, small2):
        sch.submit(r)
    plan = sch.plan()
    # big takes 6 of 8 pages; small1 (4 pages) does not fit; small2 would, but must wait behind small1
    assert [r.rid for r, _, _ in plan.portions] == [0] and [r.rid for r in sch.queue] == [1, 2]


def test_submit_refuses_what_can_never_fit():
    sch, cache = make(pages=4, page_size=4, max_len=64)
    with pytest.raises(ValueError, match="capacity of 16"):
        sch.submit(req(0, 10, 7))
    with pytest.raises(ValueError, match="empty prompt"):
        sch.submit(req(1, 0, 2))
    sch.submit(req(2, 10, 6))


def test_out_of_pages_the_most_junior_steps_back_and_recomputes():
    sch, cache = make(pages=6, page_size=4, max_len=24, max_num_seqs=4, max_prefill_tokens=16)
    a, b = req(0, 8, 14), req(1, 8, 6)
    sch.submit(a); sch.submit(b)
    plans = run(sch, cache, [a, b])
    assert sch.evictions >= 1 and a.evictions == 0 and b.evictions >= 1, "the most senior never loses its pages"
    assert len(a.generated) == 14 and len(b.generated) == 6
    # after stepping back, b's known tokens (prompt and output so far) are recomputed as one portion
    back = next(i for i, p in enumerate(plans) if p.evicted)
    again = next(p for p in plans[back + 1:] if any(r is b for r, _, _ in p.portions))
    r, start, n = next(x for x in again.portions if x[0] is b)
    assert start == 0 and n > 8, "the output so far is recomputed with the prompt"


def test_victims_go_most_junior_first_and_return_to_their_place_in_line():
    sch, cache = make(pages=8, page_size=4, max_len=32, max_num_seqs=4, max_prefill_tokens=32)
    a, b, c = req(0, 7, 20), req(1, 7, 4), req(2, 7, 4)
    for r in (a, b, c):
        sch.submit(r)
    late = req(3, 3, 2)
    order_of_eviction = []
    step = 0
    while sch.has_unfinished():
        if step == 3:
            sch.submit(late)
        plan = sch.plan()
        step += 1
        order_of_eviction += [v.rid for v in plan.evicted]
        if plan.evicted:
            assert [r.rid for r in sch.queue] == sorted(r.rid for r in sch.queue), "an evicted request queues ahead of later arrivals"
        for w in plan.work:
            r = w.request
            r.cached += w.count
            cache.commit(r.rid, r.cached)
            if r.cached == r.known:
                r.generated.append(7)
                if len(r.generated) >= r.params.max_tokens:
                    sch.retire(r, "length")
        assert step < 500
    assert order_of_eviction and order_of_eviction[0] == 2 and 0 not in order_of_eviction


def test_a_lone_decoder_steps_back_itself_when_nothing_junior_holds_pages():
    sch, cache = make(pages=4, page_size=4, max_len=16, max_num_seqs=2, max_prefill_tokens=16)
    a, b = req(0, 7, 8), req(1, 7, 8)
    sch.submit(a); sch.submit(b)
    run(sch, cache, [a, b])
    assert len(a.generated) == 8 and len(b.generated) == 8 and sch.evictions >= 1


def test_prefill_first_runs_portions_alone_but_not_forever():
    sch, cache = make(pages=64, max_len=128, max_num_seqs=4, max_prefill_tokens=4, prefill_first=2)
    a, b = req(0, 2, 30), req(1, 40, 2)
    sch.submit(a)
    plans = run(sch, cache, [a, b], arrivals={2: b})
    k = kinds(plans)
    assert "pp" in k and "ppp" not in k[2:], k
    assert sch.steps_held_back == sum(1 for p in plans if p.held_back) > 0


def test_mixed_prefill_tokens_caps_portions_only_while_someone_decodes():
    sch, cache = make(pages=64, max_len=128, max_num_seqs=4, max_prefill_tokens=16, mixed_prefill_tokens=3)
    a, b = req(0, 2, 40), req(1, 30, 2)
    sch.submit(a)
    plans = run(sch, cache, [a, b], arrivals={2: b})
    with_decode = [sum(n for _, _, n in p.portions) for p in plans if p.decode and p.portions]
    assert with_decode and max(with_decode) == 3
    # alone, a prompt takes the full budget
    sch2, cache2 = make(pages=64, max_len=128, max_num_seqs=4, max_prefill_tokens=16, mixed_prefill_tokens=3)
    c = req(0, 30, 2)
    sch2.submit(c)
    assert [n for _, _, n in run(sch2, cache2, [c])[0].portions] == [16]


def test_prefill_every_lets_portions_in_on_every_nth_step_only():
    sch, cache = make(pages=64, max_len=128, max_num_seqs=4, max_prefill_tokens=4, prefill_every=3)
    a, b = req(0, 2, 40), req(1, 20, 2)
    sch.submit(a)
    plans = run(sch, cache, [a, b], arrivals={2: b})
    mixed_steps = [i + 1 for i, p in enumerate(plans) if p.decode and p.portions]
    assert mixed_steps and all(s % 3 == 0 for s in mixed_steps)
    assert len(b.generated) == 2


def test_max_prefill_seqs_bounds_the_portions_of_a_step():
    sch, cache = make(pages=64, max_len=128, max_num_seqs=6, max_prefill_tokens=64, max_prefill_seqs=2)
    rs = [req(i, 5, 2) for i in range(5)]
    for r in rs:
        sch.submit(r)
    plans = run(sch, cache, rs)
    assert [len(p.portions) for p in plans[:3]] == [2, 2, 1]
    free, cache_free = make(pages=64, max_len=128, max_num_seqs=6, max_prefill_tokens=64)
    rs = [req(i, 5, 2) for i in range(5)]
    for r in rs:
        free.submit(r)
    assert len(run(free, cache_free, rs)[0].portions) == 5


def test_the_token_budget_bounds_decoded_rows_too():
    sch, cache = make(pages=64, max_len=128, max_num_seqs=6, max_prefill_tokens=64, max_num_batched_tokens=3)
    rs = [req(i, 2, 6) for i in range(5)]
    for r in rs:
        sch.submit(r)
    plans = run(sch, cache, rs)
    assert max(p.num_tokens for p in plans) == 3 and all(len(r.generated) == 6 for r in rs)


@pytest.mark.parametrize("seed", range(8))
def test_random_load_finishes_and_keeps_invariants(seed):
    rng = random.Random(seed)
    knobs = {}
    if seed % 2:
        knobs = dict(prefill_first=rng.choice((0, 1, 3)), prefill_every=rng.choice((1, 2)),
                     mixed_prefill_tokens=rng.choice((None, 5)), max_prefill_seqs=rng.choice((None, 2)))
    sch, cache = make(pages=24, page_size=4, max_len=64, max_num_seqs=5, max_prefill_tokens=rng.choice((8, 16, 64)), **knobs)
    reqs, arrivals, t = [], {}, 0
    for i in range(14):
        n, m = rng.randint(1, 40), rng.randint(1, 20)
        r = req(i, n, m)
        reqs.append(r)
        t += rng.choice((0, 0, 1, 3))
        while t in arrivals:
            t += 1
        arrivals[t] = r
    plans = run(sch, cache, reqs, arrivals)
    work = sum(len(r.prompt) + r.params.max_tokens for r in reqs)
    assert all(r.phase is Phase.DONE and len(r.generated) == r.params.max_tokens for r in reqs)
    assert len(plans) <= 2 * work + 2 + max(arrivals), "no starvation"
    assert reqs[0].evictions == 0, "the most senior request never loses its pages"
