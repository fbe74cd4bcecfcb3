"""The scheduler's decisions with a scripted step instead of a model (no GPU): admission,
portions under the token budget, decoding, finishing and freeing, and what happens when
pages run out.  The method follows the reference's `SteppedModel` tests
(rust/engine/src/runner/model_runner.rs:987-1106, 1209-2683)."""

from llm_inference_lab_b200.cache import CacheManager, GroupConfig
from llm_inference_lab_b200.cache.manager import runtime


def make(pages=64, page_size=4, max_requests=8, budget=8, reserve_future=True, max_seq_len=0, window=0):
    cache = CacheManager([GroupConfig(page_size, window, pages)], max_requests)
    sched = runtime().Scheduler(cache, budget, max_seq_len, 0, reserve_future)
    return cache, sched


def run(sched, next_token=lambda rid, pos: 100 + rid, max_steps=10_000):
    """Drives the scheduler to the end; returns (plans, {id: Finished})."""
    plans, done = [], {}
    for _ in range(max_steps):
        plan = sched.plan()
        for f in sched.take_finished():
            done[f.id] = f
        if not plan:
            assert sched.idle, "requests are left but nothing is planned"
            break
        plans.append([(e.id, e.start, e.n, e.sample) for e in plan])
        sampled = [next_token(e.id, e.start + e.n) for e in plan if e.sample]
        sched.complete(plan, sampled)
        for f in sched.take_finished():
            done[f.id] = f
    return plans, done


def test_one_request_prefill_then_decode():
    cache, sched = make(budget=8)
    sched.add(1, list(range(5)), 3)
    plans, done = run(sched)
    assert plans == [[(1, 0, 5, True)], [(1, 5, 1, True)], [(1, 6, 1, True)]]
    assert done[1].generated == [101, 101, 101] and done[1].reason.name == "length"
    assert cache.free_pages(0) == 64 and cache.live_requests == 0, "the last token needs no cache entry"


def test_prompt_is_cut_into_portions_under_the_budget():
    cache, sched = make(budget=4)
    sched.add(1, list(range(10)), 2)
    plans, done = run(sched)
    assert plans == [[(1, 0, 4, False)], [(1, 4, 4, False)], [(1, 8, 2, True)], [(1, 10, 1, True)]]
    assert len(done[1].generated) == 2


def test_decode_tokens_come_first_and_prefill_takes_the_rest():
    cache, sched = make(budget=6)
    sched.add(1, [1, 2, 3], 4)
    plan = sched.plan()
    sched.complete(plan, [7])                          # request 1 now decodes
    sched.add(2, list(range(20)), 1)
    sched.add(3, list(range(4)), 1)
    plan = sched.plan()
    assert [(e.id, e.start, e.n, e.sample) for e in plan] == [(1, 3, 1, True), (2, 0, 5, False)]
    sched.complete(plan, [7])
    plan = sched.plan()
    assert [(e.id, e.n) for e in plan] == [(1, 1), (2, 5)], "request 3 waits for budget, in order"
    sched.complete(plan, [7])
    plans, done = run(sched)
    assert set(done) == {1, 2, 3} and cache.free_pages(0) == 64


def test_budget_one_two_three_give_the_same_tokens():
    outs = []
    for budget in (1, 2, 3, 50):
        cache, sched = make(budget=budget)
        sched.add(1, [5, 6, 7, 8, 9], 4)
        sched.add(2, [1], 3)
        _, done = run(sched, next_token=lambda rid, pos: 10 * rid + pos)
        outs.append({k: v.generated for k, v in done.items()})
    assert all(o == outs[0] for o in outs) and outs[0][2] == [21, 22, 23]


def test_eos_finishes_and_counts_the_token():
    cache, sched = make()
    sched.add(1, [1, 2], 10, eos=[42, 43])
    sched.add(2, [1, 2], 3, eos=[42], ignore_eos=True)
    toks = {1: iter([5, 43, 6]), 2: iter([42, 42, 42])}
    _, done = run(sched, next_token=lambda rid, pos: next(toks[rid]))
    assert done[1].generated == [5, 43] and done[1].reason.name == "eos"
    assert done[2].generated == [42, 42, 42] and done[2].reason.name == "length"


def test_invalid_and_trivial_requests():
    cache, sched = make(max_seq_len=16)
    sched.add(1, [], 2)
    sched.add(2, list(range(10)), 8)                   # 10 + 8 - 1 = 17 > 16
    sched.add(3, list(range(10)), 7)                   # 16: fits
    sched.add(4, [1, 2], 0)
    _, done = run(sched)
    assert done[1].reason.name == "invalid" and "empty" in done[1].message
    assert done[2].reason.name == "invalid" and "maximum sequence length" in done[2].message
    assert done[3].reason.name == "length" and len(done[3].generated) == 7
    assert done[4].reason.name == "length" and done[4].generated == []


def test_admission_protects_the_future_of_running_requests():
    """With reservation a request is admitted only if the pages for its whole life are free
    beyond what running requests will still take; a later, smaller request may pass it."""
    cache, sched = make(pages=6, page_size=4, budget=64)         # 24 tokens of cache
    sched.add(1, list(range(4)), 9)                              # life: 12 tokens = 3 pages
    sched.add(2, list(range(12)), 5)                             # life: 16 tokens = 4 pages: does not fit beside 1
    sched.add(3, list(range(5)), 4)                              # life: 8 tokens = 2 pages: fits
    plan = sched.plan()
    assert [e.id for e in plan] == [1, 3] and sched.num_waiting == 1
    sched.complete(plan, [9, 9])
    plans, done = run(sched)
    assert set(done) == {1, 2, 3} and all(f.reason.name == "length" for f in done.values())
    assert sched.preemptions == 0 and all(f.preemptions == 0 for f in done.values())
    first_of_2 = next(i for i, p in enumerate(plans) if any(e[0] == 2 for e in p))
    assert all(any(e[0] == 1 for e in p) or any(e[0] == 3 for e in p) for p in plans[:first_of_2])
    assert cache.free_pages(0) == 6


def test_request_that_can_never_fit_fails_at_once():
    cache, sched = make(pages=4, page_size=4)
    sched.add(1, list(range(30)), 1)
    sched.add(2, list(range(3)), 2)
    _, done = run(sched)
    assert done[1].reason.name == "capacity" and done[2].reason.name == "length"


def test_pages_run_out_without_reservation_youngest_is_preempted_and_recomputed():
    """Optimistic admission: both requests start, pages run out while they decode, the younger
    one gives its pages back, waits, and later recomputes prompt + tokens so far.  Every
    request still gets all its tokens, the same ones as alone."""
    def token(rid, pos):
        return 1000 * rid + pos

    alone = {}
    for rid, prompt, n in ((1, list(range(6)), 14), (2, list(range(7)), 12)):
        cache, sched = make(pages=64, budget=16, reserve_future=False)
        sched.add(rid, prompt, n)
        alone[rid] = run(sched, token)[1][rid].generated
    cache, sched = make(pages=7, page_size=4, budget=16, reserve_future=False)    # 28 tokens of cache
    sched.add(1, list(range(6)), 14)                             # grows to 19 tokens
    sched.add(2, list(range(7)), 12)                             # grows to 18 tokens
    plans, done = run(sched, token)
    assert sched.preemptions >= 1 and done[2].preemptions >= 1 and done[1].preemptions == 0
    assert done[1].generated == alone[1] and done[2].generated == alone[2]
    assert done[1].reason.name == "length" and done[2].reason.name == "length"
    recompute = [p for p in plans if any(e[0] == 2 and e[1] == 0 and e[2] > 7 for e in p)]
    assert recompute, "request 2 came back with prompt + generated tokens as one prompt"
    assert cache.free_pages(0) == 7 and cache.live_requests == 0
    cache.check_consistency()


def test_alone_and_still_too_large_fails_with_capacity():
    cache, sched = make(pages=3, page_size=4, budget=8, reserve_future=False)
    sched.add(1, list(range(6)), 20)                             # would grow to 25 tokens > 12
    _, done = run(sched)
    assert done[1].reason.name == "capacity" and 0 < len(done[1].generated) < 20
    assert cache.free_pages(0) == 3


def test_failed_step_gives_reserved_pages_back():
    cache, sched = make(pages=8, budget=16)
    sched.add(1, list(range(9)), 2)
    plan = sched.plan()
    assert cache.free_pages(0) == 5
    sched.abandon(plan)
    assert cache.free_pages(0) == 8 and cache.reserved(1) == 0
    plan = sched.plan()                                           # the same step is planned again
    assert [(e.start, e.n) for e in plan] == [(0, 9)]


def test_cancel_waiting_and_running():
    cache, sched = make()
    sched.add(1, [1, 2, 3], 5)
    sched.add(2, [1, 2, 3], 5)
    plan = sched.plan()
    sched.complete(plan, [4, 4])
    assert sched.cancel(1) and not sched.cancel(99)
    sched.add(3, [1], 1)
    assert sched.cancel(3)
    _, done = run(sched)
    assert done[1].reason.name == "cancelled" and done[3].reason.name == "cancelled"
    assert done[2].reason.name == "length" and cache.free_pages(0) == 64


def test_state_slots_bound_the_number_of_running_requests():
    cache, sched = make(max_requests=2)
    for rid in range(5):
        sched.add(rid, [1, 2], 2)
    plan = sched.plan()
    assert len(plan) == 2 and sched.num_waiting == 3
    sched.complete(plan, [0, 0])
    _, done = run(sched)
    assert len(done) == 5 and cache.free_state_slots == 2


def test_windowed_group_is_budgeted_by_its_peak():
    cache, sched = make(pages=6, page_size=4, window=6, budget=4)
    sched.add(1, list(range(40)), 20)            # 59 tokens, far more than 24 slots, but the window needs 4 pages
    _, done = run(sched)
    assert done[1].reason.name == "length" and len(done[1].generated) == 20
    assert cache.free_pages(0) == 6


# ----------------------------------------------------------------------------------------
# Lookahead: the next decode step is planned while the last one's tokens are still unknown.
# ----------------------------------------------------------------------------------------

def run_ahead(sched, next_token, max_steps=10_000):
    """As `run`, but decode steps are planned ahead whenever the scheduler allows it: the tokens of
    step n reach `complete` only after step n + 1 has been planned (as they do when the device feeds
    them forward).  Returns (plans, {id: Finished}, number of steps planned ahead)."""
    plans, done, ahead_count = [], {}, 0

    def collect():
        for f in sched.take_finished():
            done[f.id] = f

    for _ in range(max_steps):
        plan = sched.plan()
        collect()
        if not plan:
            assert sched.idle
            break
        while True:
            plans.append([(e.id, e.start, e.n, e.sample) for e in plan])
            pure = all(e.n == 1 and e.sample for e in plan)
            ahead = sched.plan_ahead(plan) if pure else []
            sampled = [next_token(e.id, e.start + e.n) for e in plan if e.sample]
            sched.complete(plan, sampled)
            collect()
            if not ahead:
                break
            ahead_count += 1
            plan = ahead
    return plans, done, ahead_count


def test_lookahead_gives_the_same_tokens_and_frees_everything():
    import random

    rng = random.Random(4)
    looked_ahead = 0
    for trial in range(40):
        n_req = rng.randint(1, 6)
        reqs = [(i + 1, [rng.randint(0, 50) for _ in range(rng.randint(1, 30))], rng.randint(1, 25))
                for i in range(n_req)]
        stop_at = {rid: rng.randint(2, 40) for rid, _, _ in reqs}       # position at which each samples its EOS

        def token(rid, pos):
            return 999 if pos >= stop_at[rid] + len(reqs[rid - 1][1]) else 100 + (rid * 7 + pos) % 50

        results = []
        for mode in ("plain", "ahead"):
            cache, sched = make(pages=200, page_size=4, budget=16)
            for rid, prompt, max_new in reqs:
                sched.add(rid, prompt, max_new, [999], False)
            if mode == "plain":
                _, done = run(sched, token)
                used = 0
            else:
                _, done, used = run_ahead(sched, token)
            assert cache.free_pages(0) == 200 and cache.live_requests == 0
            cache.check_consistency()
            results.append(({rid: (f.generated, f.reason.name) for rid, f in done.items()}, used))
        assert results[0][0] == results[1][0], f"trial {trial}"
        looked_ahead += results[1][1]
    assert looked_ahead > 100, "most decode steps were planned ahead"


def test_lookahead_plans_the_next_position_and_stops_before_the_last_token():
    cache, sched = make(budget=8)
    sched.add(1, [1, 2, 3], 4)
    sched.add(2, [4, 5], 6)
    plan = sched.plan()                                   # both prompts
    assert sched.plan_ahead(plan) == [], "a step with prompt portions is not looked ahead from"
    sched.complete(plan, [10, 20])
    plan = sched.plan()                                   # first decode step: positions 3 and 2
    assert [(e.id, e.start) for e in plan] == [(1, 3), (2, 2)]
    ahead = sched.plan_ahead(plan)
    assert [(e.id, e.start, e.n, e.sample) for e in ahead] == [(1, 4, 1, True), (2, 3, 1, True)]
    sched.complete(plan, [11, 21])
    # request 1 has 2 of its 4 tokens; the step in flight gives the third, the one after it the last
    ahead2 = sched.plan_ahead(ahead)
    assert [(e.id, e.start) for e in ahead2] == [(1, 5), (2, 4)]
    sched.complete(ahead, [12, 22])
    assert sched.plan_ahead(ahead2) == [], "request 1 ends by length with the step in flight"
    sched.complete(ahead2, [13, 23])
    done = {f.id: f for f in sched.take_finished()}
    assert done[1].generated == [10, 11, 12, 13] and done[1].reason.name == "length"
    assert sched.num_active == 1


def test_a_request_that_ends_while_the_next_step_runs_leaves_with_that_step():
    cache, sched = make(budget=8)
    sched.add(1, [1, 2, 3], 10, [99], False)
    sched.add(2, [4, 5], 10, [99], False)
    sched.complete(sched.plan(), [10, 20])
    plan = sched.plan()
    ahead = sched.plan_ahead(plan)
    assert ahead
    held = cache.free_pages(0)
    sched.complete(plan, [99, 21])                         # request 1 samples its end-of-sequence token
    assert sched.num_active == 2 and cache.free_pages(0) == held, "it stays until the step in flight is done"
    assert sched.take_finished() == []
    assert sched.plan_ahead(ahead) == [], "no further lookahead while a request is on its way out"
    sched.complete(ahead, [55, 22])                        # its token of this step is dropped
    done = {f.id: f for f in sched.take_finished()}
    assert done[1].generated == [10, 99] and done[1].reason.name == "eos"
    assert sched.num_active == 1 and cache.free_pages(0) > held
    plan = sched.plan()
    assert [(e.id, e.start) for e in plan] == [(2, 4)]
    assert sched.portion(2, 4, 1) == [22]


def test_lookahead_waits_when_requests_are_waiting_or_pages_are_short():
    cache, sched = make(pages=3, page_size=4, budget=8, reserve_future=False)      # 12 tokens of cache
    sched.add(1, list(range(7)), 8)
    sched.complete(sched.plan(), [50])
    plan = sched.plan()                                   # position 7: the second page is full after it
    ahead = sched.plan_ahead(plan)
    assert [(e.id, e.start) for e in ahead] == [(1, 8)], "the third page is there"
    sched.complete(plan, [51])
    sched.add(2, [1, 2], 2)                               # someone waits: admission comes first
    assert sched.plan_ahead(ahead) == []
    sched.complete(ahead, [52])
    cache.check_consistency()


def test_lookahead_without_a_free_page_falls_back_to_the_plain_plan():
    cache, sched = make(pages=2, page_size=4, budget=8, reserve_future=False)      # 8 tokens of cache
    sched.add(1, list(range(7)), 8)
    sched.complete(sched.plan(), [50])
    plan = sched.plan()                                   # position 7 fills the second page
    assert sched.plan_ahead(plan) == [], "no page for position 8"
    sched.complete(plan, [51])                            # the step in flight still completes as ever
    cache.check_consistency()
    assert sched.plan() == [], "alone and out of pages: the request ends"
    done = {f.id: f for f in sched.take_finished()}
    assert done[1].reason.name == "capacity" and done[1].generated == [50, 51]
    assert cache.free_pages(0) == 2 and cache.live_requests == 0


# ----------------------------------------------------------------------------------------
# Random workloads: pools of every tightness, both admission policies, windows, late arrivals.
# ----------------------------------------------------------------------------------------

def test_random_workloads_give_the_scripted_tokens_and_every_page_back():
    """The scripted step answers with a token that depends on request and position only, so whatever
    the scheduler decides (portions, waiting, preemption and recomputation, lookahead), a request
    that finishes must have exactly the tokens it would have alone; one that fails with `capacity`
    must be one that cannot fit alone; and every page and state slot comes back."""
    import random

    outcomes = {"length": 0, "eos": 0, "capacity": 0, "invalid": 0, "preemptions": 0}
    for trial in range(250):
        rng = random.Random(trial)
        page = rng.choice([1, 2, 4, 8, 16])
        window = rng.choice([0, 0, 0, 5, 17])
        reqs = [(i + 1, [rng.randint(0, 50) for _ in range(rng.randint(1, 40))], rng.randint(0, 30))
                for i in range(rng.randint(1, 9))]
        life = [len(p) + max(n, 1) - 1 for _, p, n in reqs]
        biggest = max(-(-n // page) for n in life)
        pages = rng.randint(max(1, biggest - 1), max(sum(-(-n // page) for n in life), biggest) + 2)
        budget = rng.choice([1, 2, 3, 8, 16, 64])
        reserve = rng.random() < 0.5
        max_seq = rng.choice([0, 0, 45, 70])
        ahead_on = rng.random() < 0.6
        eos_on = rng.random() < 0.6
        stop = {rid: rng.randint(1, 35) for rid, _, _ in reqs}

        def token(rid, pos):
            if eos_on and pos >= stop[rid] + len(reqs[rid - 1][1]):
                return 999
            return 100 + (rid * 7 + pos) % 50

        groups = [GroupConfig(page, 0, pages)] + ([GroupConfig(page, window, pages)] if window else [])
        cache = CacheManager(groups, rng.randint(1, 9))
        sched = runtime().Scheduler(cache, budget, max_seq, 0, reserve)
        late = [(rid, p, n, [999], False) for rid, p, n in reqs][::-1]
        for _ in range(rng.randint(0, len(late))):
            sched.add(*late.pop())
        done = {}

        def collect():
            for f in sched.take_finished():
                assert f.id not in done, "a request finishes once"
                done[f.id] = f

        for _ in range(100_000):
            while late and rng.random() < 0.3:
                sched.add(*late.pop())
            plan = sched.plan()
            collect()
            if not plan:
                if late:
                    sched.add(*late.pop())
                    continue
                assert sched.idle, "requests are left but nothing is planned"
                break
            while True:
                assert sum(e.n for e in plan) <= budget
                pure = all(e.n == 1 and e.sample for e in plan)
                ahead = sched.plan_ahead(plan) if (pure and ahead_on) else []
                sched.complete(plan, [token(e.id, e.start + e.n) for e in plan if e.sample])
                collect()
                if not ahead:
                    break
                plan = ahead
        where = f"trial {trial}"
        assert set(done) == {rid for rid, _, _ in reqs}, where
        for rid, prompt, n in reqs:
            f = done[rid]
            want = []
            for i in range(n):
                want.append(token(rid, len(prompt) + i))
                if want[-1] == 999:
                    break
            reason = f.reason.name
            outcomes[reason] += 1
            outcomes["preemptions"] += f.preemptions
            if reason in ("length", "eos"):
                assert list(f.generated) == want, where
                assert reason == ("eos" if want and want[-1] == 999 else "length"), where
            elif reason == "invalid":
                assert max_seq and len(prompt) + max(n, 1) - 1 > max_seq, where
            else:
                assert reason == "capacity" and -(-(len(prompt) + max(n, 1) - 1) // page) > pages, where
                assert list(f.generated) == want[: len(f.generated)], where
        assert all(cache.free_pages(g) == pages for g in range(len(groups))) and cache.live_requests == 0, where
        cache.check_consistency()
    assert outcomes["preemptions"] > 100 and outcomes["capacity"] > 5 and outcomes["invalid"] > 20, outcomes


def test_decoding_requests_never_outnumber_the_budget():
    """A request decodes only after a portion of its prompt ran, and prompts get what the decoding
    requests leave of the budget: so the decoding requests of a step never exceed the budget, none
    of them is ever left out of a step, and a small budget only delays the prompts behind them (the
    reference's order, batch_policy.rs:36-87).  The tokens equal those of an unconstrained run."""
    outs = []
    for budget in (2, 3, 64):
        cache, sched = make(budget=budget)
        for rid in range(5):
            sched.add(rid, [1, 2][: 1 + rid % 2], 6)
        plans, done = run(sched, next_token=lambda rid, pos: 10 * rid + pos)
        outs.append({k: v.generated for k, v in done.items()})
        running = set()
        for p in plans:
            assert sum(n for _, _, n, _ in p) <= budget
            decoding = {rid for rid, start, n, sample in p if rid in running}
            assert decoding == running, "a decoding request was left out of a step"
            for rid, start, n, sample in p:
                if sample:
                    running.add(rid)
            running -= {rid for rid in running if any(e[0] == rid and e[1] + e[2] >= len([1, 2][: 1 + rid % 2]) + 5
                                                      for e in p)}
        assert cache.free_pages(0) == 64
    assert outs[0] == outs[1] == outs[2]
