"""The scheduler's decisions: admission, portions under a token budget, decode rows first,
finishing, and what happens when pages run out (the newest running request is preempted
and recomputed; a request that cannot fit even alone fails)."""
import pytest

from imparo_b200.cache import CacheManager
from imparo_b200.engine.scheduler import Scheduler
from imparo_b200.parts.spec import PagedKV, SlotState

SPECS = [(0, (PagedKV(2, 16),)), (1, (SlotState((2, 8)),))]


def make(pages=64, page=4, slots=4, budget=8, ctx=256):
    cm = CacheManager(SPECS, page, pages, slots, device=None)
    return cm, Scheduler(cm, budget, slots, ctx)


def run_step(s, plan, eos=()):
    s.step_done(True)
    finished = []
    for e in plan:
        if e.want and s.on_token(e.request, e.request in eos):
            finished.append(e.request)
    return finished


def test_prompt_is_cut_under_the_budget_and_first_token_comes_from_the_last_portion():
    cm, s = make(budget=8)
    a = s.submit(19, 3)
    plans = []
    while s.has_work():
        p = s.plan()
        plans.append([(e.request, e.start, e.count, e.want) for e in p])
        run_step(s, p)
    assert plans == [[(a, 0, 8, False)], [(a, 8, 8, False)], [(a, 16, 3, True)], [(a, 19, 1, True)], [(a, 20, 1, True)]]
    # 3 new tokens cost 2 decode steps (imparo-server/src/main.rs:1786-1790)
    assert cm.n_requests() == 0 and cm.free_pages(0) == 64 and cm.free_slots() == 4
    cm.check()


def test_decode_rows_come_first_and_share_the_step_with_portions():
    cm, s = make(budget=8)
    a = s.submit(3, 10)
    run_step(s, s.plan())                       # a: whole prompt, first token
    b = s.submit(20, 2)
    p = s.plan()
    assert [(e.request, e.start, e.count, e.want) for e in p] == [(a, 3, 1, True), (b, 0, 7, False)]
    run_step(s, p)
    p = s.plan()
    assert [(e.request, e.count) for e in p] == [(a, 1), (b, 7)]
    run_step(s, p)
    p = s.plan()
    assert [(e.request, e.start, e.count, e.want) for e in p] == [(a, 5, 1, True), (b, 14, 6, True)]
    cm.check()


def test_several_prompts_in_flight_fifo():
    cm, s = make(budget=10)
    a, b, c = s.submit(4, 2), s.submit(4, 2), s.submit(30, 2)
    p = s.plan()
    assert [(e.request, e.count, e.want) for e in p] == [(a, 4, True), (b, 4, True), (c, 2, False)]


def test_finish_by_eos_and_by_length_frees_everything():
    cm, s = make()
    a, b = s.submit(5, 4), s.submit(6, 50)
    p = s.plan(); run_step(s, p)
    assert s.n_running == 2
    p = s.plan(); fin = run_step(s, p, eos={b})
    assert fin == [b]
    for _ in range(2):
        p = s.plan(); fin = run_step(s, p)
    assert fin == [a] and not s.has_work()
    assert cm.free_pages(0) == 64 and cm.free_slots() == 4
    cm.check()


def test_admission_waits_for_a_slot_and_for_pages():
    cm, s = make(pages=6, slots=2, budget=16)
    a, b, c = s.submit(8, 8), s.submit(8, 8), s.submit(2, 2)
    p = s.plan()
    assert [e.request for e in p] == [a, b]       # no third slot
    run_step(s, p)
    assert s.n_waiting == 1
    # a and b now hold 2 pages each; each needs a third page at position 8
    p = s.plan()
    assert [e.request for e in p] == [a, b] and cm.free_pages(0) == 0
    run_step(s, p)
    cm.check()


def test_pages_run_out_newest_is_preempted_and_recomputed():
    cm, s = make(pages=6, slots=3, budget=16, page=4)
    a = s.submit(8, 20)
    run_step(s, s.plan())                         # a holds 2 pages, 9 tokens known
    b = s.submit(7, 20)
    p = s.plan()                                  # a decodes (3rd page); b: 2 pages + 1 spare <= 3 free
    assert [(e.request, e.count) for e in p] == [(a, 1), (b, 7)]
    run_step(s, p)
    assert cm.free_pages(0) == 1
    for _ in range(10):                           # b takes the last page at position 8; a needs one at 12
        p = s.plan()
        if s.n_preemptions:
            break
        assert [e.request for e in p] == [a, b]
        run_step(s, p)
    # a (older) could not get its page: the NEWEST running request, b, gave up what it held
    assert s.n_preemptions == 1 and s.take_preempted() == [b]
    assert [e.request for e in p] == [a] and cm.cached(a) == 12
    assert s.n_running == 1 and s.n_waiting == 1
    assert s.known_tokens(b) > 7                  # prompt plus what it generated so far
    run_step(s, p)
    cm.check()
    # a runs on alone; b comes back once pages are free and recomputes from position 0
    seen_b_restart = False
    for _ in range(200):
        if not s.has_work():
            break
        p = s.plan()
        for e in p:
            if e.request == b and e.start == 0:
                seen_b_restart = True
        run_step(s, p)
        cm.check()
    assert seen_b_restart and not s.has_work()
    assert cm.free_pages(0) == 6 and cm.free_slots() == 3


def test_a_request_that_cannot_fit_alone_fails_and_frees():
    cm, s = make(pages=3, slots=2, budget=8, page=4)
    a = s.submit(30, 4)                           # needs 8 pages, the pool has 3
    failed = []
    for _ in range(20):
        if not s.has_work():
            break
        p = s.plan()
        failed += s.take_failed()
        if p:
            run_step(s, p)
    assert failed == [a] and not s.has_work()
    assert cm.free_pages(0) == 3 and cm.free_slots() == 2
    cm.check()


def test_failed_step_abandons_its_requests():
    cm, s = make()
    a, b = s.submit(5, 4), s.submit(6, 4)
    p = s.plan()
    s.step_done(False)                            # imparo-server/src/sched.rs:652-660
    assert sorted(s.take_failed()) == [a, b] and not s.has_work()
    assert cm.free_pages(0) == 64 and cm.free_slots() == 4
    cm.check()


def test_refused_requests():
    cm, s = make(ctx=16)
    with pytest.raises(ValueError):
        s.submit(0, 4)
    with pytest.raises(ValueError):
        s.submit(17, 4)
    with pytest.raises(ValueError):
        s.submit(4, 0)


def test_context_limit_ends_a_request():
    cm, s = make(ctx=12, budget=16)
    a = s.submit(10, 100)
    n = 0
    while s.has_work():
        run_step(s, s.plan()); n += 1
    assert n == 2 and cm.free_pages(0) == 64      # 10 -> 11 -> 12 known: stop


def test_abort_in_the_middle_of_a_prompt_gives_everything_back():
    """A request cancelled while its prompt is still entering in portions: slot and pages go back at once,
    the others go on (the reference forgets a failed request and returns what it held:
    imparo-server/src/sched.rs:857-883)."""
    cm, s = make(pages=64, page=4, slots=3, budget=8)
    a, b = s.submit(30, 4), s.submit(5, 4)
    p = s.plan()
    assert [(e.request, e.count) for e in p] == [(a, 8)]
    run_step(s, p)
    p = s.plan()                                     # a's second portion is planned (pages reserved)
    assert (p[0].request, p[0].start, p[0].count) == (a, 8, 8)
    assert s.abort(a) == -2                          # part of the planned step: not now
    run_step(s, p)
    assert cm.cached(a) == 16 and cm.free_pages(0) == 64 - 4 and cm.free_slots() == 2
    assert s.abort(a) == 0                           # between steps: released
    assert not cm.has(a) and cm.free_pages(0) == 64 and cm.free_slots() == 3
    assert s.abort(a) == -1                          # unknown by now
    p = s.plan()
    assert [(e.request, e.start, e.count, e.want) for e in p] == [(b, 0, 5, True)]
    while s.has_work():
        run_step(s, s.plan())
    assert cm.n_requests() == 0 and cm.free_pages(0) == 64 and cm.free_slots() == 3
    cm.check()


def test_abort_of_a_waiting_request():
    cm, s = make(slots=1, budget=8)
    a, b = s.submit(4, 2), s.submit(4, 2)
    run_step(s, s.plan())
    assert s.n_waiting == 1 and s.abort(b) == 0 and s.n_waiting == 0
    while s.has_work():
        run_step(s, s.plan())
    assert cm.n_requests() == 0
    cm.check()


_PREEMPTIONS_SEEN = []


@pytest.mark.parametrize("seed", range(12))
def test_a_planned_row_never_needs_a_token_older_than_the_step_in_flight(seed):
    """What Engine.generate's pipelined loop relies on.  It reads a step's sampled ids only after the NEXT step
    has been issued.  So when it plans, the only values it lacks are those the step in flight is sampling,
    and the plan must ask for such a value only as the single token of a one-token row of the very request
    that wanted it; in particular a request that is preempted is never planned again before its
    last token has reached the host.  Random lengths, budgets and pools small enough to force preemptions;
    requests end by stop tokens (found one step late, as in the engine) and by length."""
    import random
    rng = random.Random(seed)
    page, slots = rng.choice([2, 4]), rng.choice([2, 3, 5])
    pages = rng.randint(14, 40)
    cm, s = make(pages=pages, page=page, slots=slots, budget=rng.choice([4, 8, 16]), ctx=120)
    host_known = {}                                  # request -> tokens whose values the host holds
    for _ in range(rng.randint(4, 10)):
        n = rng.randint(1, min(40, (pages - slots) * page))
        host_known[s.submit(n, rng.randint(1, 12))] = n
    in_flight = []                                   # requests whose sampled id is still on the device
    dead = set()
    steps = 0
    while s.has_work() or in_flight:
        p = s.plan() if s.has_work() else []
        for r in s.take_failed():
            host_known.pop(r, None)
        if p:
            for e in p:
                need = e.start + e.count
                if need > host_known[e.request]:
                    assert e.count == 1 and e.start == host_known[e.request] and e.request in in_flight, \
                        (seed, steps, e, host_known[e.request], in_flight)
            s.step_done(True)
        # the ids of the step before are read now, while the step just issued runs
        for r in in_flight:
            if r in dead:
                continue
            if rng.random() < 0.08:                  # it was a stop token
                dead.add(r)
                assert s.abort(r) in (0, -1)         # never -2: nothing is planned between step_done and plan
            elif r in host_known:                    # (a request that failed alone meanwhile is gone)
                host_known[r] += 1
        in_flight = []
        for e in p:
            if e.want:
                in_flight.append(e.request)
                if e.request not in dead:
                    s.on_token(e.request, False)     # optimistic, as the engine books it
        steps += 1
        assert steps < 5000
    assert cm.n_requests() == 0 and cm.free_pages(0) == pages and cm.free_slots() == slots
    cm.check()
    _PREEMPTIONS_SEEN.append(s.n_preemptions)
    if seed == 11:
        assert sum(_PREEMPTIONS_SEEN) > 0            # the pools were small enough to matter


def test_padded_rows_rule_and_budget():
    """The step function fills the one-token rows up to 1, 2, 4, 8, 16, 24, ... rows; a scheduler told so counts
    those rows in its token budget, so a step with prompt portions holds exactly the budget while prompts are left."""
    from imparo_b200.engine.scheduler import padded_rows
    assert [padded_rows(n) for n in (0, 1, 2, 3, 4, 5, 8, 9, 16, 17, 31, 33)] == [0, 1, 2, 4, 4, 8, 8, 16, 16, 24, 32, 40]
    cm = CacheManager([(0, (PagedKV(1, 8, None),))], page_size=4, num_pages=4000, num_slots=12)
    budget = 64
    s = Scheduler(cm, budget, 12, 1000, count_padded_rows=True)
    plain = Scheduler(CacheManager([(0, (PagedKV(1, 8, None),))], page_size=4, num_pages=4000, num_slots=12), budget, 12, 1000)
    for sched in (s, plain):
        for n in (5, 9, 30, 200, 7, 300, 11, 250, 400):
            sched.submit(n, 40)
    seen = set()
    for _ in range(60):
        plan = s.plan()
        if not plan:
            break
        ones = sum(1 for e in plan if e.count == 1)
        total = sum(e.count for e in plan)
        padded = total + padded_rows(ones) - ones
        assert padded <= budget
        if s.n_waiting > 0 or any(e.count > 1 and not e.want for e in plan):
            assert padded == budget, (ones, total)          # prompts are left: the step is full to the row
        seen.add(ones)
        s.step_done(True)
        for e in plan:
            if e.want:
                s.on_token(e.request, False)
    assert len(seen) > 3
    # without the option the budget counts real tokens only
    p = plain.plan()
    assert sum(e.count for e in p) == budget
