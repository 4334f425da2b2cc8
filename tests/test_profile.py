"""The per-step profile's bookkeeping (no GPU: events are faked): the time between two consecutive marks of a step is
booked to the later one's class, steps do not bleed into each other, and the report gives shares and bytes / time."""
from fusezap_core_b200.kernels.profile import StepProfile, contexts, format_report, ideal_linear_bytes


class FakeEvent:
    clock = 0.0

    def __init__(self):
        self.at = None

    def record(self):
        FakeEvent.clock += 0.25
        self.at = FakeEvent.clock

    def elapsed_time(self, other):
        return other.at - self.at


def test_profile_books_time_between_marks():
    FakeEvent.clock = 0.0
    p = StepProfile(FakeEvent)
    for _ in range(4):
        p.begin_step()
        p.note("norm", 1000)
        p.note("linear", 8_000_000)
        p.note("norm", 1000)
        FakeEvent.clock += 10.0            # host time between steps is nobody's
    p.collect(lambda: None)
    rep = p.report()
    rows = {r["class"]: r for r in rep["classes"]}
    assert rep["steps"] == 4 and abs(rep["ms"] - 3.0) < 1e-9
    assert rows["norm"]["launches"] == 8 and abs(rows["norm"]["ms"] - 2.0) < 1e-9 and abs(rows["norm"]["share"] - 2 / 3) < 1e-3
    assert rows["linear"]["ideal_bytes"] == 32_000_000 and rows["linear"]["ideal_gbs"] == 32.0
    text = format_report(rep)
    assert "norm" in text and "linear" in text and "4 steps" in text
    p.collect(lambda: None)                # nothing new: totals stay
    assert p.report()["steps"] == 4


def test_ideal_bytes_helpers():
    assert ideal_linear_bytes(8, 4096, 4096, 2, 2, 4) == 8 * 4096 * 2 + 4096 * 4096 * 2 + 8 * 4096 * 4

    class Seg:
        def __init__(self, n, pos0): self.n, self.pos0 = n, pos0
    # one decoded token at position 99 sees 100 keys; a portion of 3 from position 10 sees 11 + 12 + 13
    assert contexts([Seg(1, 99), Seg(3, 10)]) == 100 + 36


def test_timeline_costs_from_timestamps():
    """`per_launch_costs`: per position in a step, the median over the steps of (next launch's dependency met - this
    launch's dependency met) and of (dependency met - first block started)."""
    from fusezap_core_b200.kernels.timeline import per_launch_costs
    events = []
    t = 1000
    for step in range(3):
        # three launches per step: costs 5, 7 + step (so the median is 8) and a last one that has no successor in its step
        for name, start_before, cost in (("rowwise", 2, 5), ("gemm_tc", 10, 7 + step), ("attn_decode", 4, 30)):
            events.append((t - start_before * 1000, t, name))
            t += cost * 1000
    rows = per_launch_costs(events, 3)
    assert [r["file"] for r in rows] == ["rowwise", "gemm_tc", "attn_decode"]
    assert rows[0]["cost_us"] == 5.0 and rows[1]["cost_us"] == 8.0 and rows[2]["cost_us"] != rows[2]["cost_us"]      # nan
    assert [r["resident_before_us"] for r in rows] == [2.0, 10.0, 4.0]
