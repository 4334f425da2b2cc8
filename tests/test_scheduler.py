"""The scheduler's decisions alone (no model): a fake token function drives it, and after every step the invariants
are checked, in the manner of the reference's tests/test_scheduler.py:26-135."""
import random

import pytest
import torch

from fusezap_core_b200.cache import CacheManager, KVNeed
from fusezap_core_b200.engine.scheduler import Scheduler, SchedulerConfig, Sequence, SeqStatus


class P:   # what the scheduler needs of sampling params
    def __init__(self, max_tokens): self.max_tokens = max_tokens


def make(pages=16, page_size=4, max_len=64, **cfg):
    cache = CacheManager({0: KVNeed(1, 16, 0)}, {}, page_size, pages, 8, max_len, torch.float32, "cpu", allocate=False)
    return Scheduler(SchedulerConfig(**cfg), cache), cache


def run(sch, cache, seqs, arrivals=None, max_steps=2000):
    """Drives the scheduler as the engine does. Returns the list of SchedulerOutputs."""
    outs, pending = [], sorted(arrivals.items()) if arrivals else []
    step = 0
    while sch.has_unfinished() or pending:
        while pending and pending[0][0] <= step:
            s = pending.pop(0)[1]
            sch.add(s, s.params.max_tokens)
        so = sch.schedule()
        step += 1
        assert step < max_steps, "the scheduler does not finish"
        rows = [(s, s.num_computed, 1) for s in so.decode] + list(so.prefill)
        # invariants of one step
        assert len({id(s) for s, _, _ in rows}) == len(rows), "a request twice in one step"
        assert so.num_tokens <= sch.cfg.token_budget
        assert sum(n for _, _, n in so.prefill) <= sch.cfg.max_prefill_tokens
        assert len(sch.running) <= sch.cfg.max_num_seqs
        for v in so.preempted:
            assert v.num_computed == 0 and v.status == SeqStatus.WAITING and not cache.holds(v.seq_id)
            assert all(v is not s for s, _, _ in rows), "a request that lost its pages runs in the same step"
        for s, start, n in rows:
            assert start == s.num_computed and 1 <= n <= s.num_pending
            assert len(cache.table(0, s.seq_id)) * cache.page_size >= start + n, "rows without pages"
        cache.check()
        for s, start, n in rows:
            s.num_computed += n
            cache.commit(s.seq_id, s.num_computed)
            if s.num_computed == s.num_tokens:
                s.output.append(1000 + len(s.output))
                if len(s.output) >= s.params.max_tokens:
                    sch.finish(s, "length")
        outs.append(so)
    assert cache.num_free_pages == cache.num_pages
    return outs


def seq(i, n_prompt, max_tokens, arrival=None):
    return Sequence(i, list(range(n_prompt)), P(max_tokens), arrival=i if arrival is None else arrival)


def test_prompt_is_cut_into_portions_under_the_budget():
    sch, cache = make(max_num_seqs=4, max_prefill_tokens=8)
    s = seq(0, 20, 3)
    sch.add(s, 3)
    outs = run(sch, cache, [s])
    assert [[(n) for _, _, n in o.prefill] for o in outs[:3]] == [[8], [8], [4]]
    assert [len(o.decode) for o in outs] == [0, 0, 0, 1, 1] and s.finish_reason == "length" and len(s.output) == 3


def test_portions_and_decoded_tokens_share_a_step():
    sch, cache = make(max_num_seqs=4, max_prefill_tokens=8)
    a, b = seq(0, 4, 6), seq(1, 20, 2)
    sch.add(a, 6)
    outs = run(sch, cache, [a, b], arrivals={2: b})
    mixed = [o for o in outs if o.decode and o.prefill]
    assert len(mixed) >= 2, "a prompt portion runs beside a decoded token"


def test_head_of_queue_is_never_skipped():
    sch, cache = make(pages=8, page_size=4, max_len=32, max_num_seqs=4, max_prefill_tokens=64)
    big, small1, small2 = seq(0, 24, 4), seq(1, 14, 2), seq(2, 2, 2)
    for s in (big, small1, small2):
        sch.add(s, s.params.max_tokens)
    so = sch.schedule()
    # big takes 6 of 8 pages; small1 (4 pages) does not fit; small2 would, but must wait behind small1
    assert [s.seq_id for s, _, _ in so.prefill] == [0] and [s.seq_id for s in sch.waiting] == [1, 2]


def test_add_refuses_what_can_never_fit():
    sch, cache = make(pages=4, page_size=4, max_len=64)
    with pytest.raises(ValueError, match="capacity of 16"):
        sch.add(seq(0, 10, 7), 7)
    with pytest.raises(ValueError, match="empty prompt"):
        sch.add(seq(1, 0, 2), 2)
    sch.add(seq(2, 10, 6), 6)


def test_out_of_pages_newest_steps_back_and_recomputes():
    sch, cache = make(pages=6, page_size=4, max_len=24, max_num_seqs=4, max_prefill_tokens=16)
    a, b = seq(0, 8, 14), seq(1, 8, 6)
    sch.add(a, 14); sch.add(b, 6)
    outs = run(sch, cache, [a, b])
    assert sch.num_preemptions >= 1 and a.num_preemptions == 0 and b.num_preemptions >= 1, "the oldest never loses its pages"
    assert len(a.output) == 14 and len(b.output) == 6
    # after stepping back, b's known tokens (prompt and output so far) are recomputed as one portion
    back = next(i for i, o in enumerate(outs) if o.preempted)
    again = next(o for o in outs[back + 1:] if any(s is b for s, _, _ in o.prefill))
    s, start, n = next(x for x in again.prefill if x[0] is b)
    assert start == 0 and n > 8, "the output so far is recomputed with the prompt"


def test_a_lone_decoder_steps_back_itself_when_nothing_newer_holds_pages():
    sch, cache = make(pages=4, page_size=4, max_len=16, max_num_seqs=2, max_prefill_tokens=16)
    a, b = seq(0, 7, 8), seq(1, 7, 8)
    sch.add(a, 8); sch.add(b, 8)
    run(sch, cache, [a, b])
    assert len(a.output) == 8 and len(b.output) == 8 and sch.num_preemptions >= 1


def test_prefill_first_runs_portions_alone_but_not_forever():
    sch, cache = make(pages=64, max_len=128, max_num_seqs=4, max_prefill_tokens=4, prefill_first=2)
    a, b = seq(0, 2, 30), seq(1, 40, 2)
    sch.add(a, 30)
    outs = run(sch, cache, [a, b], arrivals={2: b})
    kinds = ["p" if o.prefill and not o.decode else "d" if o.decode and not o.prefill else "m" for o in outs]
    assert "pp" in "".join(kinds) and "ppp" not in "".join(kinds[2:]), kinds


@pytest.mark.parametrize("seed", range(5))
def test_random_load_finishes_and_keeps_invariants(seed):
    rng = random.Random(seed)
    sch, cache = make(pages=24, page_size=4, max_len=64, max_num_seqs=5, max_prefill_tokens=rng.choice((8, 16, 64)))
    seqs, arrivals, t = [], {}, 0
    for i in range(14):
        n, m = rng.randint(1, 40), rng.randint(1, 20)
        s = seq(i, n, m)
        seqs.append(s)
        t += rng.choice((0, 0, 1, 3))
        while t in arrivals:
            t += 1
        arrivals[t] = s
    outs = run(sch, cache, seqs, arrivals)
    work = sum(len(s.prompt) + s.params.max_tokens for s in seqs)
    assert all(s.status == SeqStatus.FINISHED and len(s.output) == s.params.max_tokens for s in seqs)
    assert len(outs) <= 2 * work + 2 + max(arrivals), "no starvation"
    oldest_running_never_preempted = seqs[0].num_preemptions == 0
    assert oldest_running_never_preempted
