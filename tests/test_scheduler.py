"""The scheduler's decisions, on the CPU: admission, portions under a budget,
rotation, finishing, and what happens when pages run out."""
import pytest
import torch

from cellm_b200.cache import CacheManager
from cellm_b200.engine import Scheduler, SchedulerError
from cellm_b200.parts import FixedState, PagedKV


def make(pages=16, page=4, slots=3, budget=16, chunk=8, max_pos=256):
    cm = CacheManager([FixedState((2, 4)), PagedKV(1, 8, 0)], [None, None], page, pages, slots, torch.float32, "cpu")
    return cm, Scheduler(cm, budget, chunk, max_pos)


def run_step(s, token=5, stop_on=None):
    """schedule, pretend the step ran, append a token wherever logits were wanted."""
    plan = s.schedule()
    s.step_done()
    finished = []
    for e in plan.entries:
        if e.wants_logits and s.append_token(e.request_id, token, stop=(stop_on == e.request_id)):
            finished.append(e.request_id)
    return plan, finished


def test_prompts_are_cut_into_portions_under_the_budget():
    cm, s = make()
    s.add_request(0, list(range(20)), 4)
    s.add_request(1, list(range(5)), 4)
    plan, _ = run_step(s)
    assert [(e.request_id, e.start, e.count, e.wants_logits) for e in plan.entries] == [(0, 0, 8, False), (1, 0, 5, True)]
    assert sorted(r for r, _ in plan.admitted) == [0, 1]
    plan, _ = run_step(s)      # request 1 decodes first, request 0 goes on with its prompt
    assert [(e.request_id, e.start, e.count) for e in plan.entries] == [(1, 5, 1), (0, 8, 8)]
    plan, _ = run_step(s)
    assert [(e.request_id, e.start, e.count, e.wants_logits) for e in plan.entries] == [(1, 6, 1, True), (0, 16, 4, True)]
    assert s.info(0)["state"] == "decoding" and s.info(0)["generated"] == 1


def test_budget_limits_decoders_and_rotation_serves_all():
    cm, s = make(pages=32, slots=4, budget=2, chunk=2)
    for r in range(3):
        s.add_request(r, [1, 2], 50)
    served = {0: 0, 1: 0, 2: 0}
    while not all(s.info(r)["state"] == "decoding" for r in range(3)):
        run_step(s)
    for _ in range(9):
        plan, _ = run_step(s)
        assert len(plan.entries) == 2 and sum(e.count for e in plan.entries) == 2
        for e in plan.entries:
            served[e.request_id] += 1
    assert set(served.values()) == {6}          # two of three each step, evenly


def test_admission_waits_for_a_slot_and_keeps_arrival_order():
    cm, s = make(slots=2)
    for r in range(4):
        s.add_request(r, [1, 2, 3], 2)
    plan, _ = run_step(s)
    assert [r for r, _ in plan.admitted] == [0, 1] and s.stats()["waiting"] == 2
    plan, fin = run_step(s)
    assert fin == [0, 1] and s.info(0)["finish_reason"] == "length"
    plan, _ = run_step(s)
    assert [r for r, _ in plan.admitted] == [2, 3]


def test_finish_frees_pages_and_slot_stop_and_cancel():
    cm, s = make()
    s.add_request(0, list(range(6)), 10)
    s.add_request(1, list(range(6)), 10)
    run_step(s)
    assert cm.free_pages(0) == 16 - 4 and cm.free_slots == 1
    _, fin = run_step(s, stop_on=0)
    assert fin == [0] and s.info(0)["finish_reason"] == "stop"
    assert cm.free_pages(0) == 16 - 2 and cm.free_slots == 2
    s.cancel(1)
    assert s.info(1)["finish_reason"] == "cancelled" and cm.free_pages(0) == 16 and cm.free_slots == 3
    assert s.stats()["idle"]
    s.forget(0)
    assert not s.has(0)
    with pytest.raises(SchedulerError):
        s.cancel(0)


def test_requests_that_cannot_fit_are_refused_when_added():
    cm, s = make(pages=4, page=4, max_pos=64)
    with pytest.raises(SchedulerError, match="pages"):
        s.add_request(0, list(range(10)), 10)           # 20 tokens > 4 pages of 4
    with pytest.raises(SchedulerError, match="positions"):
        s.add_request(1, list(range(60)), 10)
    with pytest.raises(SchedulerError):
        s.add_request(2, [], 4)
    with pytest.raises(SchedulerError):
        s.add_request(3, [1], 0)
    s.add_request(4, list(range(10)), 6)
    with pytest.raises(SchedulerError, match="exists"):
        s.add_request(4, [1], 1)


def test_pages_run_out_newest_request_is_preempted_and_recomputed():
    cm, s = make(pages=6, page=4, slots=3, budget=32, chunk=16)
    s.add_request(0, list(range(8)), 12)     # 2 pages now, 5 in the end
    s.add_request(1, list(range(8)), 12)
    plan, _ = run_step(s)
    assert len(plan.entries) == 2 and cm.free_pages(0) == 2
    preempted_at = None
    for step in range(40):
        plan, fin = run_step(s)
        if plan.preempted:
            assert plan.preempted == [1]                    # the one admitted last
            assert not plan.admitted                        # and nobody is admitted in that step
            assert s.info(1)["state"] == "waiting" and s.info(1)["computed"] == 0
            assert s.info(1)["num_tokens"] == 8 + s.info(1)["generated"]      # it keeps what it generated
            preempted_at = step
            break
    assert preempted_at is not None
    recomputed = False
    while not s.stats()["idle"]:
        plan, fin = run_step(s)
        for e in plan.entries:      # when 1 comes back it recomputes prompt + generated, in portions that
            if e.request_id == 1 and e.start == 0:         # end at a page edge while pages are short
                recomputed = True
                assert e.count == 13 and e.wants_logits      # 8 prompt + 5 generated, admitted once all of it fits
    assert recomputed and s.info(0)["generated"] == 12 and s.info(1)["generated"] == 12
    assert s.info(1)["preemptions"] >= 1 and s.stats()["preemptions"] >= 1
    assert cm.free_pages(0) == 6 and cm.free_slots == 3


def test_prefill_that_holds_each_others_pages_is_untangled():
    cm, s = make(pages=4, page=4, slots=2, budget=8, chunk=4)
    s.add_request(0, list(range(12)), 2)
    s.add_request(1, list(range(12)), 2)
    steps = 0
    while not s.stats()["idle"]:
        run_step(s)
        steps += 1
        assert steps < 60
    assert s.info(0)["generated"] == 2 and s.info(1)["generated"] == 2 and cm.free_pages(0) == 4


def test_append_rules():
    cm, s = make()
    s.add_request(0, list(range(12)), 3)
    s.schedule()
    s.step_done()
    with pytest.raises(SchedulerError, match="not decoding"):
        s.append_token(0, 1)
    assert s.tokens(0) == list(range(12)) and s.tokens(0, 10) == [10, 11]


def test_a_model_without_paged_items_is_scheduled_by_slots_and_budget_alone():
    cm = CacheManager([FixedState((2, 4))], [None], 4, 1, 2, torch.float32, "cpu")
    s = Scheduler(cm, 16, 8, 256)
    for rid in range(3):
        s.add_request(rid, list(range(10)), 3)
    plan, _ = run_step(s)
    assert [(e.request_id, e.start, e.count) for e in plan.entries] == [(0, 0, 8), (1, 0, 8)]     # two slots
    done = []
    for _ in range(20):
        plan, fin = run_step(s)
        done += fin
        if len(done) == 3:
            break
    assert sorted(done) == [0, 1, 2] and cm.free_slots == 2 and s.stats()["preemptions"] == 0


@pytest.mark.parametrize("seed", range(24))
def test_random_arrivals_keep_the_invariants(seed):
    """Requests of random length arrive at random steps into pools of random size (often too
    small for all at once), some stop early, some are cancelled. In every step: the budget and the
    portion limit hold, every portion starts where the request's cache ends, nobody appears twice,
    pages and slots add up; in the end everybody has finished with the tokens it was given and
    everything is free."""
    import numpy as np
    rng = np.random.default_rng(seed)
    page = int(rng.choice([2, 4, 8]))
    n_req = int(rng.integers(3, 12))
    growing = seed % 2 == 1          # short prompts that grow long in a tight pool: running requests get preempted
    lens = rng.integers(1, 12 if growing else 60, n_req).tolist()
    news = rng.integers(20 if growing else 1, 60 if growing else 30, n_req).tolist()
    need = [-(-(l + n) // page) for l, n in zip(lens, news)]
    pages = int(max(max(need), sum(need) * rng.uniform(0.2, 0.6 if growing else 1.1)))
    slots = n_req if growing else int(rng.integers(1, n_req + 1))
    budget, chunk = int(rng.integers(1, 48)), int(rng.integers(1, 32))
    cm = CacheManager([FixedState((2, 4)), PagedKV(1, 8, 0)], [None, None], page, pages, slots, torch.float32, "cpu")
    s = Scheduler(cm, budget, chunk, 4096)
    arrive = sorted(rng.integers(0, 3 if growing else 40, n_req).tolist())
    stop_after = {r: int(rng.integers(1, news[r] + 1)) for r in range(n_req) if rng.random() < 0.3}
    cancel_at = {r: int(rng.integers(1, 80)) for r in range(n_req) if rng.random() < 0.15}
    given = {r: [] for r in range(n_req)}         # the tokens handed to each request, in order
    added, cancelled, finished = set(), set(), set()
    cached = {}                                   # request -> tokens in its cache, as the plans imply
    step = 0
    while len(finished | cancelled) < n_req:
        for r in range(n_req):
            if r not in added and arrive[r] <= step:
                s.add_request(r, list(range(r, r + lens[r])), news[r])
                added.add(r)
        for r, at in cancel_at.items():
            if at == step and r in added and r not in finished and r not in cancelled:
                s.cancel(r)
                cancelled.add(r)
                cached.pop(r, None)
        plan = s.schedule()
        for r in plan.preempted:
            cached.pop(r, None)                   # recomputed from the start
        seen = set()
        assert sum(e.count for e in plan.entries) <= budget
        for e in plan.entries:
            assert e.request_id not in seen and e.request_id not in finished | cancelled
            seen.add(e.request_id)
            assert 1 <= e.count <= max(chunk, 1)
            assert e.start == cached.get(e.request_id, 0), (e, cached)
            total = lens[e.request_id] + len(given[e.request_id])
            assert e.start + e.count <= total
            assert e.wants_logits == (e.start + e.count == total)
            cached[e.request_id] = e.start + e.count
        s.step_done()
        held = 0
        for r in added - finished - cancelled:
            if cm.has(r):
                n_blocks = len(cm.block_table(r, 0))
                assert n_blocks * page >= cached.get(r, 0)
                held += n_blocks
        assert held + cm.free_pages(0) == pages
        for e in plan.entries:
            if e.wants_logits:
                r = e.request_id
                tok = 1000 + len(given[r])
                given[r].append(tok)
                if s.append_token(r, tok, stop=stop_after.get(r) == len(given[r])):
                    finished.add(r)
                    cached.pop(r, None)
        step += 1
        assert step < 5000, "the scheduler stopped making progress"
    for r in finished:
        info = s.info(r)
        assert info["generated"] == len(given[r]) == stop_after.get(r, news[r])
        assert info["finish_reason"] == ("stop" if r in stop_after else "length")
        assert s.tokens(r) == list(range(r, r + lens[r])) + given[r]
    assert s.stats()["idle"] and cm.free_pages(0) == pages and cm.free_slots == slots
    PREEMPTIONS_SEEN[seed] = s.stats()["preemptions"]


PREEMPTIONS_SEEN: dict = {}


def test_random_arrivals_did_meet_preemption():
    """The random runs above are only worth their name if pages did run out in a good share of them."""
    assert len(PREEMPTIONS_SEEN) < 24 or sum(1 for v in PREEMPTIONS_SEEN.values() if v > 0) >= 6


def test_a_prompt_longer_than_a_windowed_pool_is_admitted_and_runs_through():
    """A windowed group holds a window and a portion of keys, not the prompt: a request accepted by
    that measure must also be admitted by it, or it waits for ever."""
    cm = CacheManager([PagedKV(1, 8, 0), PagedKV(1, 8, 8)], [None, None], 4, [16, 6], 2, torch.float32, "cpu")
    s = Scheduler(cm, 8, 8, 256)
    s.add_request(0, list(range(40)), 6)            # 46 tokens: 12 pages of the full group, at most 5 of the windowed one
    assert cm.pages_for(1, 46, 8) <= 6 < (46 + 3) // 4
    steps = 0
    while not s.stats()["idle"]:
        plan, _ = run_step(s)
        assert plan.entries, "a step planned nothing although a request waits"
        assert cm.free_pages(1) >= 0
        steps += 1
        assert steps < 100
    assert s.info(0)["finish_reason"] == "length" and s.info(0)["generated"] == 6
    assert cm.free_pages(0) == 16 and cm.free_pages(1) == 6 and cm.free_slots == 2
    # and what the windowed pool can never hold is refused when added, not left waiting
    with pytest.raises(SchedulerError, match="pages"):
        Scheduler(CacheManager([PagedKV(1, 8, 32)], [None], 4, [6], 2, torch.float32, "cpu"), 8, 8, 256) \
            .add_request(0, list(range(40)), 6)


def test_two_schedulers_keep_their_own_plans():
    """The planned step belongs to its scheduler: two engines stepped in turn on one thread do not mix them."""
    cm1, s1 = make()
    cm2, s2 = make()
    s1.add_request(0, list(range(5)), 3)
    s2.add_request(7, list(range(11)), 3)
    p1 = s1.schedule()
    p2 = s2.schedule()
    assert s1.plan_shape()[:2] == (1, 5) and s2.plan_shape()[:2] == (1, 8)
    assert [e.request_id for e in p1.entries] == [0] and [e.request_id for e in p2.entries] == [7]
    s1.step_done()
    s2.step_done()
    assert s1.info(0)["computed"] == 5 and s2.info(7)["computed"] == 8


def test_tokens_whose_values_come_later():
    """A step's tokens may be counted before their values are known (the engine launches the next step before it
    reads them): they are appended as pending, the next step is planned on them, and the values follow. A value that
    ends its request drops what was counted after it; a request that ended by its length keeps all its tokens."""
    cm, s = make(pages=32, slots=3, budget=16, chunk=8)
    s.add_request(0, [1, 2, 3], 4)
    s.add_request(1, [4, 5], 3)
    plan = s.schedule()
    s.step_done()
    assert s.append_rows([10, 20], [False, False]) == [False, False]          # the prompts' tokens, read at once
    # two decode steps counted ahead of their values
    for _ in range(2):
        plan = s.schedule()
        assert [(e.request_id, e.count) for e in plan.entries] == [(0, 1), (1, 1)]
        s.step_done()
        fin = s.append_pending_rows(2)
    assert fin == [False, True] and s.info(1)["state"] == "finished"          # request 1 has its three tokens
    assert s.tokens(0) == [1, 2, 3, 10, -1, -1] and s.tokens(1) == [4, 5, 20, -1, -1]
    # the plan's ids carry the pending marker: the kernels take the value from the device
    plan = s.schedule()
    assert [(e.request_id, e.start) for e in plan.entries] == [(0, 5)]
    s.step_done()
    assert s.append_pending_rows(1) == [True]                                  # and request 0 its four
    # values: the first step's, then the second's in which request 0's token ends it
    assert s.resolve_rows([0, 1], [4, 3], [11, 21], [False, False]) == [True, True]      # both have ended by their length
    assert s.resolve_rows([0, 1], [5, 4], [12, 22], [True, False]) == [True, True]
    assert s.tokens(0) == [1, 2, 3, 10, 11, 12] and s.info(0)["finish_reason"] == "stop" and s.info(0)["generated"] == 3
    assert s.tokens(1) == [4, 5, 20, 21, 22] and s.info(1)["finish_reason"] == "length"
    with pytest.raises(SchedulerError, match="no pending token"):
        s.resolve_rows([1], [4], [9], [False])                                # given already
    with pytest.raises(SchedulerError, match="no pending token"):
        s.resolve_rows([1], [1], [9], [False])                                # a prompt token
    assert s.resolve_rows([77], [0], [9], [False]) == [True]                  # a request nobody knows any more
    s.forget(0)
    s.forget(1)
    assert s.stats()["idle"] and cm.free_slots == 3 and cm.free_pages(0) == 32
    # a row whose request ended meanwhile is passed over when the step's tokens are appended
    s.add_request(2, [1, 2], 5)
    s.add_request(3, [3], 5)
    s.schedule(); s.step_done()
    assert s.append_rows([7, 8], [False, False]) == [False, False]
    s.schedule(); s.step_done()
    s.cancel(3)
    assert s.append_rows([9, -2], [False, False]) == [False, True]
    assert s.tokens(2) == [1, 2, 7, 9] and s.tokens(3) == [3, 8]
