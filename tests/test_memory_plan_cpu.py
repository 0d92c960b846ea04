"""The static memory planner (the counterpart of StaticMemoryPlanner.plan, Sources/MetalHLOCore/Memory/
StaticMemoryPlanner.swift:175-253, which the reference tests in MemoryPlanningTests.swift): no two buffers that are live
at the same step may overlap in the arena, offsets are 256-byte aligned, the arena is a multiple of 4096 and not larger
than the sum of the (aligned) sizes, and lifetime reuse actually happens. Checked on random interval sets (hypothesis) and
on the plans of real modules."""
import numpy as np
from hypothesis import given, settings
from hypothesis import strategies as st

from metalhlo_b200 import capi, modules


def check_plan(rows, arena):
    assert arena % 4096 == 0
    live = [(b, f, l, o) for b, f, l, o in rows if b > 0]
    for b, f, l, o in live:
        assert o % 256 == 0 and o >= 0 and o + b <= arena
    for i, (b1, f1, l1, o1) in enumerate(live):
        for b2, f2, l2, o2 in live[i + 1:]:
            if l1 < f2 or l2 < f1:
                continue  # never live together: may share memory
            assert o1 + b1 <= o2 or o2 + b2 <= o1, ((b1, f1, l1, o1), (b2, f2, l2, o2))
    aligned_sum = sum((b + 255) // 256 * 256 for b, *_ in live)
    assert arena <= (aligned_sum + 4095) // 4096 * 4096


interval = st.tuples(st.integers(0, 1 << 20), st.integers(0, 40), st.integers(0, 40)).map(lambda t: (t[0], min(t[1], t[2]), max(t[1], t[2])))


@settings(max_examples=200, deadline=None)
@given(st.lists(interval, min_size=0, max_size=60))
def test_live_buffers_never_overlap(intervals):
    sizes, firsts, lasts = [i[0] for i in intervals], [i[1] for i in intervals], [i[2] for i in intervals]
    offsets, arena = capi.plan_intervals(sizes, firsts, lasts)
    check_plan([(b, f, l, o) for b, f, l, o in zip(sizes, firsts, lasts, offsets)], arena)


def test_disjoint_lifetimes_share_memory_and_a_chain_needs_two_buffers():
    # a chain x0 -> x1 -> x2 -> ... where each buffer is read only by the next step: two slots are enough
    n, size = 20, 1 << 16
    offsets, arena = capi.plan_intervals([size] * n, list(range(n)), [i + 1 for i in range(n)])
    assert arena == 2 * size and len(set(offsets)) == 2
    # all live at once: no sharing possible
    offsets, arena = capi.plan_intervals([size] * 4, [0] * 4, [9] * 4)
    assert arena == 4 * size and sorted(offsets) == [0, size, 2 * size, 3 * size]
    assert capi.plan_intervals([], [], []) == ([], 0)


def test_plans_of_real_modules():
    text, _ = modules.gpt2_module(batch=2, seq=128, layers=3, d_model=256, heads=4, vocab=1031)
    for level in (0, 3):
        rows, arena = capi.plan_memory(text, level)
        assert len(rows) > 10
        check_plan(rows, arena)
        # lifetime reuse: the arena is smaller than the sum of all intermediates
        assert arena < 0.75 * sum(b for b, *_ in rows), (arena, sum(b for b, *_ in rows))
    text, _ = modules.cnn_module(batch=4, size=16, channels=3, width=16, classes=10, dt="f32")
    rows, arena = capi.plan_memory(text, 2)
    check_plan(rows, arena)
