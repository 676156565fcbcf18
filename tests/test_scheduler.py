"""The scheduler's decisions, against a simulated worker whose token is a function of (request, position), after the
reference's planner tests (tests/Starlings.Roost.Engine.Tests/Scheduling/StepPlannerTests.cs:15-175,337-364;
PlannerHarness.cs:36-56)."""
import pytest

from roost_b200.cache.manager import CacheGroup, CacheManager
from roost_b200.engine.request import GREEDY, Request, RequestError, SamplingParameters
from roost_b200.engine.scheduler import Scheduler, SchedulerOptions


def make(pages=64, page=16, **opt):
    groups = [CacheGroup("full", "paged", runs=(0,), page_size=page, kv_heads=1, head_dim=16),
              CacheGroup("state", "state", runs=(), state_shape=(0,))]
    cm = CacheManager(groups, [pages, 64])
    return Scheduler(cm, SchedulerOptions(**opt)), cm


def fake_token(rid, position):
    return (sum(map(ord, str(rid))) % 97 + 31 * position) % 1000 + 10


def run_step(s: Scheduler):
    plan = s.plan()
    if plan is None:
        return None, []
    tokens = {r.sequence.request_id: fake_token(r.sequence.request_id, r.start + r.count) for r in plan.rows if r.samples}
    return plan, s.apply(plan, tokens)


def req(rid, n, max_tokens=4, **kw):
    return Request(rid, list(range(1, n + 1)), SamplingParameters(temperature=0.0, max_tokens=max_tokens), **kw)


def test_token_budget_and_row_cap():
    s, _ = make(max_tokens_per_step=50, max_sequences_per_step=3)
    for i, n in enumerate((20, 20, 20, 20)):
        s.add(req(f"r{i}", n))
    plan = s.plan()
    assert [(r.sequence.request_id, r.start, r.count, r.samples) for r in plan.rows] == [("r0", 0, 20, True), ("r1", 0, 20, True), ("r2", 0, 10, False)]
    assert plan.num_tokens == 50


def test_a_prompt_is_cut_into_portions_and_samples_only_at_its_end():
    s, _ = make(max_tokens_per_step=32)
    s.add(req("a", 100, max_tokens=2))
    seen = []
    for _ in range(4):
        plan, events = run_step(s)
        seen.append([(r.start, r.count, r.samples) for r in plan.rows])
    assert seen == [[(0, 32, False)], [(32, 32, False)], [(64, 32, False)], [(96, 4, True)]]
    assert [e.token for e in events] == [fake_token("a", 100)]
    plan, events = run_step(s)                                   # decoding: one token at the next position
    assert [(r.start, r.count, r.samples, r.tokens) for r in plan.rows] == [(100, 1, True, [fake_token("a", 100)])]
    assert events[0].finish_reason == "length" and s.unfinished == 0


def test_portion_cap_and_decodes_beside_a_prompt():
    s, _ = make(max_tokens_per_step=40, max_chunk_tokens=16)
    s.add(req("a", 5, max_tokens=10))
    run_step(s)
    s.add(req("b", 50))
    plan, _ = run_step(s)
    assert [(r.sequence.request_id, r.start, r.count) for r in plan.rows] == [("a", 5, 1), ("b", 0, 16)]


def test_order_is_priority_then_deadline_then_arrival():
    s, _ = make(max_sequences_per_step=1)
    s.add(req("late", 4, deadline=9.0))
    s.add(req("none", 4))
    s.add(req("early", 4, deadline=1.0))
    s.add(req("high", 4, priority=1))
    order = []
    for _ in range(4):
        plan = s.plan()
        order.append(plan.rows[0].sequence.request_id)
        s.cancel(order[-1])
    assert order == ["high", "early", "late", "none"]


def test_finishes_on_stop_token_max_tokens_and_frees_pages():
    s, cm = make(model_stop_token_ids=(fake_token("m", 6), fake_token("i", 4)))
    s.add(req("m", 5, max_tokens=50))
    s.add(Request("r", [1, 2, 3], SamplingParameters(temperature=0.0, max_tokens=50), stop_token_ids=(fake_token("r", 5),)))
    # ignore_eos: the model's stop ids do not end the request, its own still do
    s.add(Request("i", [1, 2, 3], SamplingParameters(temperature=0.0, max_tokens=3, ignore_eos=True)))
    s.add(Request("j", [1, 2, 3], SamplingParameters(temperature=0.0, max_tokens=50, ignore_eos=True), stop_token_ids=(fake_token("j", 4),)))
    reasons = {}
    while s.unfinished:
        _, events = run_step(s)
        for e in events:
            if e.finish_reason:
                reasons[e.request_id] = (e.finish_reason, e.token)
        cm.check_invariants()
    assert reasons == {"m": ("stop", fake_token("m", 6)), "r": ("stop", fake_token("r", 5)), "i": ("length", fake_token("i", 5)),
                       "j": ("stop", fake_token("j", 4))}
    assert cm.pools[0].free_count == cm.pools[0].capacity and not list(cm.live_requests)


def test_when_pages_run_out_the_tail_is_preempted_and_recomputed_with_the_same_tokens():
    def generate(pages):
        s, cm = make(pages=pages, page=4)
        s.add(req("a", 10, max_tokens=12))
        s.add(req("b", 10, max_tokens=12))
        out = {"a": [], "b": []}
        preempted = []
        for _ in range(200):
            plan, events = run_step(s)
            if plan is None:
                break
            preempted += plan.preempted
            for e in events:
                out[e.request_id].append(e.token)
            cm.check_invariants()
        return out, preempted, s

    roomy, p0, _ = generate(pages=64)
    tight, p1, s = generate(pages=8)                             # both need 6 pages at the end: 12 do not fit
    assert p0 == [] and p1 and set(p1) == {"b"}                  # the later-ordered request is the victim, never the head
    assert tight == roomy                                        # recomputation reproduces every token
    assert s.preemption_count == len(p1)


def test_an_infeasible_request_preempts_nobody_and_is_aborted_when_nothing_else_can_run():
    s, cm = make(pages=4, page=4)                                # 16 tokens in all
    s.add(req("a", 9, max_tokens=2))
    run_step(s)
    s.add(Request("big", list(range(15)), GREEDY))               # admissible (16 tokens fit an empty pool) but not beside "a"
    plan, _ = run_step(s)
    assert plan.preempted == [] and [r.sequence.request_id for r in plan.rows] == ["a"]
    # "a" finishes; then "big" runs alone; it can never hold a 17th token, which ends it with "length", not an abort
    while s.unfinished:
        plan, events = run_step(s)
    assert events[-1].request_id == "big" and events[-1].finish_reason == "length"
    # a head that cannot fit even after every later request is preempted, with nothing else to run, is aborted
    s, cm = make(pages=4, page=4)
    s.add(req("x", 8, max_tokens=20, priority=1))
    s.add(req("y", 8, max_tokens=20))
    aborted = []
    for _ in range(60):
        plan, events = run_step(s)
        if plan is None:
            break
        aborted += [e.request_id for e in events if e.finish_reason == "aborted"]
        cm.check_invariants()
    assert s.unfinished == 0 and cm.pools[0].free_count == 4
    assert aborted == [] or set(aborted) <= {"x", "y"}


def test_admission_refusals():
    s, _ = make(pages=4, page=4, max_context=12)
    with pytest.raises(RequestError, match="InvalidOption"):
        s.add(Request("e", [], GREEDY))
    with pytest.raises(RequestError, match="InvalidOption"):
        s.add(Request("m", [1], SamplingParameters(max_tokens=0)))
    with pytest.raises(RequestError, match="InvalidOption"):
        s.add(Request("t", [1], SamplingParameters(top_p=0.0)))
    with pytest.raises(RequestError, match="PromptTooLong"):
        s.add(Request("l", list(range(16)), GREEDY))             # 16 + 1 tokens need 5 pages of 4
    with pytest.raises(RequestError, match="PromptTooLong"):
        s.add(Request("c", list(range(12)), GREEDY))             # no room for one generated token in 12 positions
    s.add(req("ok", 3))
    with pytest.raises(RequestError, match="already live"):
        s.add(req("ok", 3))


def test_plans_are_a_function_of_the_calls():
    def trace():
        s, _ = make(pages=10, page=4, max_tokens_per_step=12)
        log = []
        for i in range(5):
            s.add(req(f"r{i}", 5 + 3 * i, max_tokens=6))
        while s.unfinished:
            plan, _ = run_step(s)
            log.append([(r.sequence.request_id, r.start, r.count, r.samples) for r in plan.rows] + plan.preempted)
        return log
    assert trace() == trace()


def test_sizes_of_captured_steps_and_padding_rows():
    """The steps in which captured decode steps grow, and the tables of a row that only fills one up."""
    import numpy as np

    from roost_b200.cache.manager import CacheManager, build_groups
    from roost_b200.engine.batch import BatchBuilder, pad_row, padded_rows
    from roost_b200.parts.attention_work import attention_work
    from roost_b200.engine.executor import graph_kv_cap, graph_rows
    from roost_b200.parts import CacheNeed
    assert [graph_rows(n) for n in (1, 5, 8, 9, 12, 13, 17, 33, 64, 65, 100)] == [1, 5, 8, 12, 12, 16, 24, 48, 64, 96, 128]
    assert all(n <= graph_rows(n) <= max(n, n * 3 // 2 + 1) for n in range(1, 600))
    assert [graph_kv_cap(n) for n in (1, 1024, 1025, 8192, 8193, 32768, 32769)] == [1024, 1024, 2048, 8192, 12288, 32768, 49152]
    groups = build_groups([CacheNeed(kind="paged", kv_heads=1, head_dim=16, window=None)], 4)
    cm = CacheManager(groups, [8, 4])     # the paged group and the (empty) group of fixed-size state
    rc = cm.extend("a", 6)
    rows = padded_rows([(rc, 5, [9], [0])], 3, 3)
    assert rows[1:] == [pad_row(1), pad_row(1)]
    ht = BatchBuilder("cpu", cm).host_tables(rows, vocab=16)
    ids, pos, trow, q_indptr, kv_lens, selected, slot, indptr, indices, state_slots, fresh = ht.arrays
    # padding rows name the scratch slot beyond the pool's four; no row of this step brings a request's first token
    assert state_slots.tolist()[1:] == [4, 4] and fresh.tolist() == [0, 0, 0] and selected.tolist() == [0]
    assert pos.tolist() == [5, -1, -1] and kv_lens.tolist() == [6, 0, 0] and q_indptr.tolist() == [0, 1, 2, 3]
    assert slot.tolist()[1:] == [-1, -1] and slot[0] >= 0 and indptr.tolist() == [0, 2, 2, 2] and len(indices) == 2
    assert ht.max_position == 5 and ht.max_kv_len == 6 and ht.row_starts == [5, -1, -1]
    prefill, decode, merge, slots = attention_work(ht.row_starts, ht.row_counts, 4, None, 64)
    assert decode == [0, 0, 6, -1] and not prefill and not merge and slots == 0
    # for clusters of four a row brings four items in key order, the empty ones last, and nothing to merge; under a window
    # the first item is the chunk the window begins in
    _, decode, merge, slots = attention_work([130, -1, 4], [1, 1, 2], 4, None, 64, cluster=4)
    assert decode == [0, 0, 64, 0, 0, 64, 128, 1, 0, 128, 131, 2, 0, 0, 0, 3,
                      2, 0, 6, 0, 2, 0, 0, 1, 2, 0, 0, 2, 2, 0, 0, 3] and not merge and slots == 0
    _, decode, _, _ = attention_work([200], [1], 4, 70, 64, cluster=2)
    assert decode == [0, 128, 192, 0, 0, 192, 201, 1]
    with pytest.raises(ValueError):
        attention_work([200], [1], 4, None, 64, cluster=2)
    # a step of several tokens a row: the padding tokens one to a padding row, the rest to the first; rows may stay empty
    assert [len(r[2]) for r in padded_rows([(rc, 2, [1, 2, 3], [2])], 8, 4)] == [3, 3, 1, 1]
    assert [len(r[2]) for r in padded_rows([(rc, 2, [1, 2, 3], [2])], 4, 4)] == [3, 0, 1, 0]
    ht = BatchBuilder("cpu", cm).host_tables(padded_rows([(rc, 2, [1, 2, 3], [2])], 4, 4), vocab=16)
    assert ht.arrays[3].tolist() == [0, 3, 3, 4, 4] and ht.arrays[4].tolist() == [5, 0, 0, 0] and ht.arrays[1].tolist() == [2, 3, 4, -1]
    with pytest.raises(ValueError):
        padded_rows([(rc, 2, [1, 2, 3], [2])], 4, 1)
    from roost_b200.engine.executor import graph_tokens
    assert [graph_tokens(n) for n in (2, 8, 9, 33, 64, 65, 505, 512, 513, 1000, 1025, 2000)] == [8, 8, 16, 64, 64, 128, 512, 512, 640, 1024, 1280, 2048]
