"""The scheduler's decisions (no GPU).  The model is faked: the next token of a
request is a hash of all its tokens so far, so outputs do not depend on how the
work was cut — unless the scheduler feeds the wrong tokens or positions."""
import pytest

from easy_gpt.cpp_b200.cache import CacheManager
from easy_gpt.cpp_b200.engine.scheduler import Scheduler, SchedulerOptions
from easy_gpt.cpp_b200.parts.base import PagedKVNeed
from easy_gpt.cpp_b200.sampling import GREEDY

NEED = {0: PagedKVNeed(1, 8, None)}


def fake_next(tokens):
    h = 17
    for t in tokens:
        h = (h * 31 + t + 1) % 1009
    return h % 50 + 3          # never 0..2, so an EOS of 1 is only produced on purpose


def make(num_pages=64, page_size=4, **opts):
    cache = CacheManager(NEED, page_size, num_pages, opts.get("max_active", 16), 4096)
    return Scheduler(cache, SchedulerOptions(**opts)), cache


def drive(sched, cache, max_rounds=10_000, next_token=fake_next, log=None):
    fed = {}
    for _ in range(max_rounds):
        if not sched.has_work():
            return
        batch = sched.schedule()
        if not batch and not sched.has_work():
            return                      # the round only failed a request that fits nowhere
        assert batch, "has work but schedules nothing"
        assert sum(s.count for s in batch) <= sched.opt.max_batch_tokens
        assert len({s.request.id for s in batch}) == len(batch)
        tokens = []
        for s in batch:
            r = s.request
            # the step function would find exactly r.computed tokens in the cache
            assert s.start == r.computed == cache.length_of(r.id)
            fed.setdefault(r.id, []).append((s.start, s.count))
            assert s.samples == (s.start + s.count == r.known)
            if s.samples:
                tokens.append(next_token(r.tokens[:s.start + s.count]))
        if log is not None:
            log.append([(s.request.id, s.start, s.count) for s in batch])
        sched.update(batch, tokens)
        cache.check()
    raise AssertionError("did not finish")


def expected_output(prompt, n, eos=-1):
    toks, out = list(prompt), []
    for _ in range(n):
        t = fake_next(toks)
        out.append(t)
        toks.append(t)
        if t == eos:
            break
    return out


def test_portions_under_the_budget_and_decodes_first():
    sched, cache = make(max_batch_tokens=16, chunk_size=10, prefill_batch=4)
    a = sched.add(list(range(25)), GREEDY, 4)
    log = []
    drive(sched, cache, log=log)
    assert a.output == expected_output(range(25), 4)
    assert log[0] == [(0, 0, 10)] and log[1] == [(0, 10, 10)] and log[2] == [(0, 20, 5)]
    assert log[3] == [(0, 25, 1)]
    # a second request arriving later: the decoding one goes first, the prompt gets the rest of the budget
    sched, cache = make(max_batch_tokens=16, chunk_size=32, prefill_batch=4)
    a = sched.add(list(range(5)), GREEDY, 6)
    b_holder = []
    log = []

    def feed(tokens):
        if not b_holder:
            b_holder.append(sched.add(list(range(40, 70)), GREEDY, 3))
        return fake_next(tokens)

    drive(sched, cache, next_token=feed, log=log)
    assert log[1] == [(0, 5, 1), (1, 0, 15)]
    assert log[2] == [(0, 6, 1), (1, 15, 15)]
    assert a.output == expected_output(range(5), 6) and b_holder[0].output == expected_output(range(40, 70), 3)


def test_admission_limits_follow_the_reference_knobs():
    sched, cache = make(max_active=3, prefill_batch=2, max_batch_tokens=64, chunk_size=64)
    reqs = [sched.add([i + 1] * 3, GREEDY, 50) for i in range(5)]
    b1 = sched.schedule()
    assert [s.request.id for s in b1] == [0, 1]                       # at most prefill_batch admissions per round
    sched.update(b1, [fake_next(s.request.tokens) for s in b1])
    b2 = sched.schedule()
    assert [s.request.id for s in b2] == [0, 1, 2]                    # then up to max_active live
    sched.update(b2, [fake_next(s.request.tokens) for s in b2])
    b3 = sched.schedule()
    assert [s.request.id for s in b3] == [0, 1, 2] and len(sched.waiting) == 2
    assert reqs[3].state == "waiting"


def test_finish_reasons_and_freeing():
    sched, cache = make(eos_token_id=1, max_positions=12)
    by_eos = sched.add([5, 6], GREEDY, 10)
    by_length = sched.add([7, 8, 9], GREEDY, 2)
    by_positions = sched.add(list(range(10)), GREEDY, 10)
    empty = sched.add([], GREEDY, 3)
    too_long = sched.add(list(range(12)), GREEDY, 3)
    calls = {"n": 0}

    def next_token(tokens):
        calls["n"] += 1
        if tokens[:2] == [5, 6] and len(tokens) == 4:
            return 1                                                  # EOS as the third token of request 0
        return fake_next(tokens)

    drive(sched, cache, next_token=next_token)
    assert by_eos.finish_reason == "eos" and by_eos.output[-1] == 1 and len(by_eos.output) == 3   # EOS is emitted
    assert by_length.finish_reason == "length" and len(by_length.output) == 2
    assert by_positions.finish_reason == "max_positions" and len(by_positions.prompt) + len(by_positions.output) == 12
    assert empty.finish_reason == "empty" and empty.output == []
    assert too_long.finish_reason == "error" and "max_position_embeddings" in too_long.error
    assert not cache.live_requests() and cache.free_pages(0) == 64


def test_pages_run_out_newest_is_preempted_and_outputs_do_not_change():
    prompts = [[i + 1] * (9 + 3 * i) for i in range(4)]
    want = [expected_output(p, 30) for p in prompts]
    # roomy pool: no preemption
    sched, cache = make(num_pages=200, max_batch_tokens=64, chunk_size=16)
    reqs = [sched.add(p, GREEDY, 30) for p in prompts]
    drive(sched, cache)
    assert [r.output for r in reqs] == want and sched.stats.preemptions == 0
    # tight pool: 4 requests growing to 39..48 tokens need 46 pages; 24 are there
    sched, cache = make(num_pages=24, max_batch_tokens=64, chunk_size=16)
    reqs = [sched.add(p, GREEDY, 30) for p in prompts]
    log = []
    drive(sched, cache, log=log)
    assert [r.output for r in reqs] == want
    assert sched.stats.preemptions > 0
    assert reqs[0].preemptions == 0                                   # the oldest is never the victim while others run
    assert max(r.preemptions for r in reqs[1:]) > 0
    assert not cache.live_requests() and cache.free_pages(0) == 24
    # a preempted request is prefilled again from position 0 over prompt + generated tokens
    victim = max(reqs, key=lambda r: r.preemptions)
    starts = [start for step in log for rid, start, n in step if rid == victim.id]
    assert starts.count(0) == victim.preemptions + 1


def test_request_that_fits_nowhere_fails_and_the_rest_goes_on():
    sched, cache = make(num_pages=8, page_size=4)                     # 32 tokens in all
    big = sched.add(list(range(40)), GREEDY, 2)
    grows = sched.add([3] * 20, GREEDY, 30)                          # fits at first, then outgrows the pool alone
    ok = sched.add([4] * 5, GREEDY, 3)
    drive(sched, cache)
    assert big.finish_reason == "error" and "cannot fit" in big.error
    assert grows.finish_reason == "error" and "even alone" in grows.error
    assert len(grows.output) >= 12                                    # it ran until the pool was full
    assert ok.finish_reason == "length" and ok.output == expected_output([4] * 5, 3)
    assert not cache.live_requests() and cache.free_pages(0) == 8


def test_waiting_requests_keep_their_order():
    sched, cache = make(num_pages=10, page_size=4, max_batch_tokens=64, chunk_size=64)
    first = sched.add([1] * 30, GREEDY, 2)                            # 8 pages
    second = sched.add([2] * 30, GREEDY, 2)                           # must wait for pages
    third = sched.add([3] * 2, GREEDY, 2)                             # would fit, but does not overtake
    b = sched.schedule()
    assert [s.request.id for s in b] == [0]
    assert second.state == "waiting" and third.state == "waiting"
    sched.update(b, [fake_next(first.tokens)])
    drive(sched, cache)
    assert [r.id for r in sched.finished] == [0, 1, 2]


def test_tokens_in_flight_launch_then_resolve():
    """The engine launches a step before it has read the previous step's tokens: `launched` counts
    the token as existing (pending), `resolve` brings its id; outputs are the same as step by step."""
    sched, cache = make(num_pages=64, max_batch_tokens=32, chunk_size=8, eos_token_id=1)
    a = sched.add([5, 6, 7], GREEDY, 6)
    b = sched.add([9] * 11, GREEDY, 4)
    inflight = None
    rounds = 0
    while sched.has_work():
        rounds += 1
        assert rounds < 100
        batch = sched.schedule()
        if not batch:
            assert inflight is not None          # everything waits for a token on its way
            sched.resolve(*inflight)
            inflight = None
            continue
        for s in batch:
            if s.request.pending:
                assert s.count == 1              # only a decode may run on a token the host has not seen
        # tokens the "device" computes: it knows every id, pending or not
        full = {s.request.id: s.request.prompt + s.request.output + ([inflight[1][[x.request.id for x in inflight[0] if x.samples].index(s.request.id)]]
                                                                      if s.request.pending else []) for s in batch}
        tokens = [fake_next(full[s.request.id][:s.start + s.count]) for s in batch if s.samples]
        sched.launched(batch)
        if inflight is not None:
            sched.resolve(*inflight)
        inflight = (batch, tokens)
        cache.check()
    if inflight is not None:
        sched.resolve(*inflight)
    assert a.output == expected_output([5, 6, 7], 6) and b.output == expected_output([9] * 11, 4)
    assert a.finish_reason == "length" and b.finish_reason == "length" and a.pending == 0
    assert not cache.live_requests()


def test_scheduled_entries_say_whether_a_token_is_still_on_the_device():
    sched, cache = make(num_pages=64, max_batch_tokens=32)
    a = sched.add([5, 6, 7], GREEDY, 4)
    first = sched.schedule()
    assert [(s.start, s.count, s.samples, s.pending) for s in first] == [(0, 3, True, 0)]
    sched.launched(first)
    assert a.pending == 1 and a.computed == 3 and a.known == 4
    second = sched.schedule()                                 # decodes the token that has not been read yet
    assert [(s.start, s.count, s.samples, s.pending) for s in second] == [(3, 1, True, 1)]
    with pytest.raises(ValueError, match="still on the device"):
        a.token_slice(3, 1)
    sched.launched(second)
    assert sched.resolve(first, [11]) == [] and a.output == [11] and a.pending == 1
    assert sched.resolve(second, [12]) == [] and a.output == [11, 12] and a.pending == 0


def test_tokens_decoded_outside_the_scheduler_and_forgetting():
    sched, cache = make(num_pages=64)
    a = sched.add([1, 2, 3, 4], GREEDY, 10)
    sched.update(sched.schedule(), [9])
    # a loop of its own decodes three more tokens: it feeds 9, x, y and commits them
    for _ in range(3):
        cache.reserve(a.id, 1)
        cache.commit(a.id, 1)
    sched.advance_decoded(a, [21, 22, 23])
    assert a.output == [9, 21, 22, 23] and a.computed == cache.length_of(a.id) == 7 and a.known == 8
    batch = sched.schedule()
    assert [(s.start, s.count) for s in batch] == [(7, 1)]
    sched.update(batch, [30])
    while sched.has_work():
        b = sched.schedule()
        sched.update(b, [31] * sum(s.samples for s in b))
    assert a.state == "finished" and a.finish_reason == "length" and len(a.output) == 10
    assert [r.id for r in sched.finished] == [a.id]
    sched.forget(a)
    assert sched.finished == []
    with pytest.raises(KeyError):
        a.state
    with pytest.raises(ValueError):
        sched.advance_decoded(a, [1])


from hypothesis import given, settings, strategies as st  # noqa: E402


@settings(max_examples=60, deadline=None)
@given(st.lists(st.tuples(st.integers(1, 60), st.integers(1, 20)), min_size=1, max_size=10),
       st.integers(6, 60), st.sampled_from([2, 4, 8]), st.integers(3, 70), st.integers(2, 40), st.integers(1, 5), st.integers(1, 4))
def test_random_workloads_end_with_the_outputs_of_an_undisturbed_run(work, num_pages, page_size, budget, chunk, active, admit):
    """Whatever the limits: every request either fails because it cannot fit even alone or ends with exactly the
    tokens it would have got alone, every round keeps the budget, and in the end nothing is held."""
    sched, cache = make(num_pages=num_pages, page_size=page_size, max_batch_tokens=budget, chunk_size=chunk,
                        max_active=active, prefill_batch=admit)
    reqs = [sched.add([(7 * i + j) % 50 + 3 for j in range(n)], GREEDY, new) for i, (n, new) in enumerate(work)]
    drive(sched, cache)
    pool_tokens = num_pages * page_size
    for r, (n, new) in zip(reqs, work):
        assert r.state == "finished"
        if r.error:
            assert n + new > pool_tokens                      # only a request that outgrows the whole pool may fail
            assert r.output == expected_output(r.prompt, len(r.output))
        else:
            assert r.output == expected_output(r.prompt, new)
    assert not cache.live_requests() and cache.free_pages(0) == num_pages
    st_ = sched.stats
    assert st_.finished + st_.failed == len(reqs)
