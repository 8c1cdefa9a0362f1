"""The scheduler's decisions, driven with a fake step function (no GPU).

The cases follow the reference's batcher tests (crates/scheduler/src/batcher.rs:478-806):
its StubModel wrote a one-hot logit at a scripted next token; here the fake "model" is a
function from (request id, position) to the next token.
"""
import random

import pytest

from ferrum_b200 import host
from ferrum_b200.errors import InvalidRequest, NotFound, SchedulerError


def make(pages=64, page_size=4, max_requests=4, budget=16, chunk=0, eos=-1, vocab=100, window=0, width=64,
         max_model_len=0, max_seqs=256):
    h = host.module()
    cache = h.CacheManager([h.GroupSpec(page_size, window, pages, width)], max_requests)
    cfg = h.SchedulerConfig()
    cfg.max_batch_tokens, cfg.chunk_size, cfg.n_vocab = budget, chunk, vocab
    cfg.eos_token_ids = list(eos) if isinstance(eos, (list, tuple)) else ([] if eos < 0 else [eos])
    cfg.max_model_len, cfg.max_batch_seqs = max_model_len, max_seqs
    return h.Scheduler(cache, cfg), cache


def run(sched, cache, next_token=lambda rid, pos: 7, max_steps=1000, log=None):
    """Steps until idle; returns {id: [tokens]}, {id: reason}."""
    out, reasons = {}, {}
    for _ in range(max_steps):
        if sched.idle():
            break
        plan = sched.plan()
        if log is not None:
            log.append([(p.id, p.pos0, list(p.tokens), p.sample) for p in plan])
        for p in plan:
            assert cache.seq_len(p.slot) == p.pos0                      # the model's precondition
            assert cache.pages_missing(p.slot, p.pos0 + len(p.tokens)) == [0]
        sampled = [next_token(p.id, p.pos0 + len(p.tokens) - 1) for p in plan if p.sample]
        for ev in sched.commit(sampled):
            if ev.kind == 0:
                out.setdefault(ev.id, []).append(ev.token)
            else:
                reasons[ev.id] = ev.reason
        assert cache.check() == ""
    assert sched.idle()
    return out, reasons


def test_rejects_bad_requests():
    s, _ = make()
    with pytest.raises(InvalidRequest, match="prompt must not be empty"):      # batcher.rs:57-67
        s.submit(1, [], 4)
    with pytest.raises(InvalidRequest, match="top_p"):
        s.submit(1, [1], 4, 0.0, 0.0)
    with pytest.raises(InvalidRequest, match="top_p other than 1"):
        s.submit(1, [1], 4, 0.7, 0.9)
    with pytest.raises(InvalidRequest, match="temperature"):
        s.submit(1, [1], 4, -1.0)
    with pytest.raises(InvalidRequest, match="vocabulary"):
        s.submit(1, [100], 4)
    with pytest.raises(InvalidRequest, match="exceeds"):
        s.submit(1, [1] * 200, 100)
    s.submit(1, [1, 2], 4, 0.8, 1.0, 3)                                        # temperature is accepted here
    with pytest.raises(InvalidRequest, match="already"):
        s.submit(1, [3], 1)
    with pytest.raises(NotFound):
        s.cancel(99)


def test_prefill_samples_first_token_without_reforwarding_the_prompt_tail():
    """batcher.rs:506-557."""
    s, c = make(budget=64)
    s.submit(5, [10, 11, 12], 3)
    log = []
    out, reasons = run(s, c, lambda rid, pos: 40 + pos, log=log)
    assert log[0] == [(5, 0, [10, 11, 12], True)]
    assert log[1] == [(5, 3, [42], True)] and log[2] == [(5, 4, [43], True)]
    assert out == {5: [42, 43, 44]} and reasons == {5: host.module().FINISH_LENGTH} and len(log) == 3


def test_eos_and_stop_tokens_are_emitted_then_finish_with_stop():
    """batcher.rs:560-591."""
    s, c = make(eos=9)
    s.submit(1, [1, 2], 10)
    s.submit(2, [1, 2], 10, 0.0, 1.0, 0, [33])
    out, reasons = run(s, c, lambda rid, pos: {1: {1: 5, 2: 9}, 2: {1: 33}}[rid].get(pos, 0))
    assert out == {1: [5, 9], 2: [33]}
    assert reasons == {1: host.module().FINISH_STOP, 2: host.module().FINISH_STOP}
    assert c.free_slots() == 4 and c.free_pages(0) == 64


def test_any_of_several_end_tokens_stops_a_sequence():
    """A model may name several ids that end a sequence (an end-of-text and an end-of-turn id):
    whichever is drawn first is emitted and finishes the request with reason stop."""
    s, c = make(eos=[9, 17])
    s.submit(1, [1, 2], 10)
    s.submit(2, [1, 2], 10)
    out, reasons = run(s, c, lambda rid, pos: {1: {1: 5, 2: 17}, 2: {1: 6, 2: 7, 3: 9}}[rid].get(pos, 0))
    assert out == {1: [5, 17], 2: [6, 7, 9]}
    assert reasons == {1: host.module().FINISH_STOP, 2: host.module().FINISH_STOP}


def test_max_new_tokens_zero_finishes_with_length_and_no_token():
    """batcher.rs:594-613."""
    s, c = make()
    s.submit(3, [1, 2, 3], 0)
    log = []
    out, reasons = run(s, c, log=log)
    assert out == {} and reasons == {3: host.module().FINISH_LENGTH}
    assert log == [[(3, 0, [1, 2, 3], False)]]


def test_decodes_come_before_prefill_inside_the_budget():
    """batcher.rs:682-732: with a budget of 1 the decoding sequence runs, the prompt waits."""
    s, c = make(budget=1)
    s.submit(1, [4], 3)
    plan = s.plan(); s.commit([7])
    assert [(p.id, list(p.tokens)) for p in plan] == [(1, [4])]
    s.submit(2, [5, 6], 2)
    plan = s.plan()
    assert [(p.id, list(p.tokens)) for p in plan] == [(1, [7])]              # decode first, budget spent
    s.commit([7])
    s.cancel(1)
    plan = s.plan()
    assert [(p.id, p.pos0, list(p.tokens), p.sample) for p in plan] == [(2, 0, [5], False)]
    s.commit([])
    assert c.check() == ""


def test_prompts_are_cut_into_portions_under_budget_and_chunk_size():
    s, c = make(budget=10, chunk=4)
    s.submit(1, list(range(1, 12)), 2)          # 11 tokens
    s.submit(2, list(range(20, 27)), 2)         # 7 tokens
    log = []
    out, _ = run(s, c, log=log)
    assert log[0] == [(1, 0, [1, 2, 3, 4], False), (2, 0, [20, 21, 22, 23], False)]     # several prompts per step
    assert log[1] == [(1, 4, [5, 6, 7, 8], False), (2, 4, [24, 25, 26], True)]
    assert log[2] == [(2, 7, [7], True), (1, 8, [9, 10, 11], True)]                     # decode first
    assert all(sum(len(t) for _, _, t, _ in step) <= 10 for step in log)
    assert out == {1: [7, 7], 2: [7, 7]}


def test_admission_stops_when_slots_run_out():
    """batcher.rs:735-758."""
    s, c = make(max_requests=2)
    for i in range(4):
        s.submit(i, [1, 2], 1)
    s.plan()
    assert s.active() == 2 and s.queued() == 2
    s.commit([7, 7])
    out, reasons = run(s, c)
    assert set(reasons) == {2, 3}


def test_abandoned_step_leaves_every_sequence_as_before():
    """batcher.rs:761-806: a failed step must not stick."""
    s, c = make()
    s.submit(1, [1, 2, 3], 2)
    p1 = [(p.id, p.pos0, list(p.tokens)) for p in s.plan()]
    s.abandon()
    assert c.seq_len(0) == 0
    p2 = [(p.id, p.pos0, list(p.tokens)) for p in s.plan()]
    assert p1 == p2
    with pytest.raises(SchedulerError):
        s.plan()
    with pytest.raises(SchedulerError, match="number of sampled"):
        s.commit([])
    out, _ = run_from_planned(s, c)
    assert out == {1: [7, 7]}


def run_from_planned(s, c):
    s.abandon()
    return run(s, c)


def test_preemption_when_pages_run_out():
    """Two sequences decode in a pool that cannot hold both to the end: the younger one is
    preempted, recomputed later, and both produce exactly the tokens they would alone."""
    s, c = make(pages=6, page_size=4, budget=64)         # 24 tokens of cache
    s.submit(1, [1, 2, 3, 4, 5, 6], 12)                  # needs 18
    s.submit(2, [9, 8, 7, 6, 5, 4], 12)                  # needs 18
    tok = lambda rid, pos: (rid * 31 + pos * 7) % 90
    log = []
    out, reasons = run(s, c, tok, log=log)
    assert out[1] == [tok(1, 5 + i) for i in range(12)] and out[2] == [tok(2, 5 + i) for i in range(12)]
    assert s.stats().preemptions >= 1
    # the preempted sequence came back as one prompt holding what it had seen and said
    restarts = [e for step in log for e in step if e[0] == 2 and e[1] == 0]
    assert len(restarts) >= 2 and len(restarts[-1][2]) > 6 and restarts[-1][2][:6] == [9, 8, 7, 6, 5, 4]
    assert c.free_pages(0) == 6 and c.free_slots() == 4


def test_prompts_holding_each_others_pages_do_not_deadlock():
    s, c = make(pages=5, page_size=4, budget=6, chunk=3)
    s.submit(1, list(range(1, 15)), 1)                   # 14 tokens = 4 pages
    s.submit(2, list(range(21, 35)), 1)
    out, reasons = run(s, c)
    assert out == {1: [7], 2: [7]}


def test_a_request_that_can_never_fit_is_refused_at_submit():
    s, c = make(pages=4, page_size=4)
    with pytest.raises(InvalidRequest, match="exceeds"):
        s.submit(1, [1] * 10, 10)
    s.submit(2, [1] * 10, 6)
    out, _ = run(s, c)
    assert len(out[2]) == 6


@pytest.mark.parametrize("seed", range(6))
def test_random_workloads_finish_with_the_tokens_each_request_would_get_alone(seed):
    rng = random.Random(seed)
    eos = rng.choice([-1, 50])
    s, c = make(pages=rng.choice([12, 20, 40]), page_size=rng.choice([2, 4, 8]), max_requests=rng.choice([2, 3, 5]),
                budget=rng.choice([3, 8, 33]), chunk=rng.choice([0, 2, 5]), eos=eos)
    tok = lambda rid, pos: (rid * 13 + pos * 5 + seed) % 97
    want = {}
    cap = c.capacity_tokens()
    for rid in range(12):
        n, new = rng.randint(1, 20), rng.randint(0, 15)
        if n + new > cap:
            continue
        s.submit(rid, [rng.randrange(97) for _ in range(n)], new)
        exp = []
        for i in range(new):
            exp.append(tok(rid, n - 1 + i))
            if exp[-1] == eos:
                break
        want[rid] = exp
    out, reasons = run(s, c, tok, max_steps=5000)
    for rid, exp in want.items():
        assert out.get(rid, []) == exp, rid
    assert set(reasons) == set(want)
    assert c.free_pages(0) == c.group(0).num_pages and c.check() == ""


# ---------------------------------------------------------------- a step planned ahead
def run_ahead(sched, cache, next_token, max_steps=5000, log=None):
    """The engine's loop with one step planned ahead: the batch that follows is asked for before
    the current one's tokens are known, and is 'launched' with the ids of its first rows unknown."""
    out, reasons = {}, {}
    in_flight = None       # sampled rows (request id, position) of a batch that was launched ahead
    aheads = 0
    end = {}               # request id -> one past the last position of every batch launched so far
    for _ in range(max_steps):
        if sched.idle() and in_flight is None:
            break
        if in_flight is None:
            plan = sched.plan()
            if not plan:
                for ev in sched.commit([]):
                    assert ev.kind == 1
                    reasons[ev.id] = ev.reason
                continue
            end = {}                   # (an ordinary plan may have preempted: everything starts from the committed lengths)
            for p in plan:
                assert cache.seq_len(p.slot) == p.pos0 and not p.from_device
                end[p.id] = p.pos0 + len(p.tokens)
            in_flight = [(p.id, p.pos0 + len(p.tokens) - 1) for p in plan if p.sample]
        rows, in_flight = in_flight, None
        ahead = sched.plan_ahead()
        if ahead:
            aheads += 1
            dev = [a for a in ahead if a.from_device]
            assert ahead[:len(dev)] == dev or [a.id for a in ahead[:len(dev)]] == [a.id for a in dev]   # they come first
            assert [a.id for a in dev] == [r[0] for r in rows]              # this step's sampled rows, same order
            for a, (_, last_pos) in zip(dev, rows):
                assert list(a.tokens) == [-1] and a.sample
                assert a.pos0 == last_pos + 1 > cache.seq_len(a.slot)         # right after the uncommitted step
            for a in ahead:
                assert a.pos0 == end.get(a.id, cache.seq_len(a.slot))          # every batch goes on where the last ended
                assert a.from_device or all(t >= 0 for t in a.tokens)         # a prompt's tokens are known
                assert cache.pages_missing(a.slot, a.pos0 + len(a.tokens)) == [0]        # its pages are reserved
                end[a.id] = a.pos0 + len(a.tokens)
            assert sum(len(a.tokens) for a in ahead) <= 33
            in_flight = [(a.id, a.pos0 + len(a.tokens) - 1) for a in ahead if a.sample]
            if log is not None:
                log.append([a.id for a in ahead])
        # the GPU computes every launched row, also rows that turn out void; ids are passed for all
        sampled = [next_token(rid, pos) for rid, pos in rows]
        for ev in sched.commit(sampled):
            if ev.kind == 0:
                out.setdefault(ev.id, []).append(ev.token)
            else:
                reasons[ev.id] = ev.reason
                end.pop(ev.id, None)
        assert cache.check() == ""
    assert sched.idle() and in_flight is None
    return out, reasons, aheads


def test_plan_ahead_continues_a_decoding_batch_and_voids_rows_that_stop():
    s, c = make(eos=50)
    s.submit(1, [1, 2, 3], 6)
    s.submit(2, [4, 5], 6)
    tok = lambda rid, pos: 50 if (rid, pos) == (2, 3) else 7          # request 2 draws EOS as its third token
    log = []
    out, reasons, aheads = run_ahead(s, c, tok, log=log)
    assert out == {1: [7] * 6, 2: [7, 7, 50]}
    assert reasons == {1: 1, 2: 0}
    # ahead of the prompts' step and of two decode steps both rows were queued; the row of request 2
    # in the third of them was void; with one request left the plan went ahead again
    assert log[:3] == [[1, 2], [1, 2], [1, 2]] and [1] in log
    assert c.free_pages(0) == c.group(0).num_pages


def test_plan_ahead_declines_when_the_next_batch_is_not_decided():
    s, c = make(budget=4)
    s.submit(1, [1, 2, 3, 4, 5, 6], 3)              # six prompt tokens, four per step
    assert s.plan_ahead() == []                      # nothing planned
    plan = s.plan()
    ahead = s.plan_ahead()                           # a prompt portion: the rest of the prompt follows, and samples
    assert not plan[0].sample and [(a.pos0, list(a.tokens), a.sample, a.from_device) for a in ahead] == [(4, [5, 6], True, False)]
    s.commit([])
    assert s.planned()
    s.submit(2, [9], 2)
    assert s.plan_ahead() == []                      # someone is queued: the next batch admits them
    s.abandon()
    s, c = make()
    s.submit(1, [1, 2], 2)
    s.plan()
    assert [a.pos0 for a in s.plan_ahead()] == [2]   # first token now, the second one follows
    assert s.plan_ahead() == []                      # asked twice
    s.commit([7])
    assert s.planned()                               # the batch planned ahead is the plan now
    assert s.plan_ahead() == []                      # its token is the last one
    evs = s.commit([8])
    assert [(e.kind, e.token) for e in evs] == [(0, 8), (1, -1)]
    assert s.idle() and c.free_pages(0) == c.group(0).num_pages


def test_plan_ahead_leaves_a_shortage_of_pages_to_the_ordinary_plan():
    s, c = make(pages=3, page_size=2, max_requests=2)
    s.submit(1, [1, 2], 4)
    s.submit(2, [3, 4], 4)
    s.plan()                                         # a page each for the prompts, one page free
    assert s.plan_ahead() == []                      # both would need a new page
    s.commit([7, 7])
    out, reasons, _ = run_ahead(s, c, lambda rid, pos: 7)
    assert sorted(reasons) == [1, 2] and c.check() == ""


def test_cancel_while_a_batch_is_in_flight_voids_its_row():
    s, c = make()
    s.submit(1, [1, 2], 5)
    s.submit(2, [3], 5)
    s.plan()
    assert len(s.plan_ahead()) == 2
    with pytest.raises(SchedulerError, match="plan_ahead"):
        s.cancel(2)
    s.commit([7, 7])
    s.cancel(2)                                      # its row of the batch in flight is void now
    evs = s.commit([8, 9])
    assert [(e.id, e.token) for e in evs if e.kind == 0] == [(1, 8)]
    assert s.active() == 1 and c.check() == ""


@pytest.mark.parametrize("seed", range(6))
def test_random_workloads_with_steps_planned_ahead(seed):
    rng = random.Random(100 + seed)
    eos = rng.choice([-1, 50])
    s, c = make(pages=rng.choice([12, 20, 40]), page_size=rng.choice([2, 4, 8]), max_requests=rng.choice([2, 3, 5]),
                budget=rng.choice([3, 8, 33]), chunk=rng.choice([0, 2, 5]), eos=eos)
    tok = lambda rid, pos: (rid * 13 + pos * 5 + seed) % 97
    want = {}
    cap = c.capacity_tokens()
    for rid in range(12):
        n, new = rng.randint(1, 20), rng.randint(0, 15)
        if n + new > cap:
            continue
        s.submit(rid, [rng.randrange(97) for _ in range(n)], new)
        exp = []
        for i in range(new):
            exp.append(tok(rid, n - 1 + i))
            if exp[-1] == eos:
                break
        want[rid] = exp
    out, reasons, aheads = run_ahead(s, c, tok)
    for rid, exp in want.items():
        assert out.get(rid, []) == exp, rid
    assert set(reasons) == set(want)
    assert c.free_pages(0) == c.group(0).num_pages and c.check() == ""


def test_plan_ahead_mixes_the_rows_that_sample_with_the_next_portions():
    """Request 1 is decoding, request 2 has a long prompt cut into portions of 4: every step that
    is planned ahead brings request 1's next token (its id still on the GPU) first and request 2's
    next portion after it; the step in which the prompt ends samples for both."""
    s, c = make(budget=8, chunk=4)
    s.submit(1, [1, 2], 20)
    s.submit(2, list(range(10, 23)), 5)              # 13 prompt tokens
    plan = s.plan()
    assert [(p.id, len(p.tokens), p.sample) for p in plan] == [(1, 2, True), (2, 4, False)]
    ahead = s.plan_ahead()
    assert [(a.id, a.pos0, list(a.tokens), a.sample, a.from_device) for a in ahead] == \
        [(1, 2, [-1], True, True), (2, 4, [14, 15, 16, 17], False, False)]
    s.commit([7])
    ahead = s.plan_ahead()
    assert [(a.id, a.pos0, len(a.tokens), a.sample, a.from_device) for a in ahead] == [(1, 3, 1, True, True), (2, 8, 4, False, False)]
    s.commit([7])
    ahead = s.plan_ahead()                           # the last portion: one token, and it samples
    assert [(a.id, a.pos0, list(a.tokens), a.sample, a.from_device) for a in ahead] == \
        [(1, 4, [-1], True, True), (2, 12, [22], True, False)]
    s.commit([7])
    ahead = s.plan_ahead()                           # both decode now, in the order in which they sampled
    assert [(a.id, a.pos0, a.from_device) for a in ahead] == [(1, 5, True), (2, 13, True)]
    evs = s.commit([7, 8])
    assert [(e.id, e.token) for e in evs] == [(1, 7), (2, 8)]
    s.abandon()                                      # (the batch planned ahead never ran; the loop below plans afresh)
    out, reasons, _ = run_ahead(s, c, lambda rid, pos: 9)
    assert len(out[1]) + 4 == 20 and len(out[2]) + 1 == 5 and c.check() == ""
