"""The scheduler's decisions, with a fake step function and the real cache bookkeeping (no GPU)."""
import random
import zlib

import pytest

from fakes import llama_like_manager
from sharpinference_b200.engine.scheduler import FINISHED, RUNNING, WAITING, Request, Scheduler
from sharpinference_b200.sampling import SamplingParams


def next_token(tokens):
    """What the fake model 'generates' after a token sequence: a function of the sequence alone."""
    return zlib.crc32(bytes(str(list(tokens)), "ascii")) % 97 + 3


class FakeRunner:
    """Takes pages like the step function does and answers with ``next_token``."""

    def __init__(self, cache):
        self.cache = cache
        self.steps = []

    def run(self, plan):
        self.cache.reserve([(e.request.request_id, e.count) for e in plan.entries])
        sampled = []
        for e in plan.entries:
            assert self.cache.get(e.request.request_id).length == e.start
            self.cache.commit(e.request.request_id, e.count)
            if e.want_last:
                sampled.append(next_token(e.request.tokens[:e.start + e.count]))
        self.steps.append([(e.request.request_id, e.start, e.count, e.want_last) for e in plan.entries])
        self.cache.check_invariants()
        return sampled


def make(num_pages=64, page_size=4, max_batch=4, budget=16, chunk=8):
    cache = llama_like_manager(num_pages=num_pages, page_size=page_size, chunk=chunk, max_requests=max_batch)
    return cache, Scheduler(cache, max_batch=max_batch, max_tokens_per_step=budget), FakeRunner(cache)


def req(rid, n_prompt, max_new=4, stop=()):
    return Request(rid, [((rid + 1) * 7 + i) % 90 + 3 for i in range(n_prompt)],
                   SamplingParams(temperature=0.0, max_new_tokens=max_new), stop_set=tuple(stop))


def drive(sched, runner, limit=2000):
    done = []
    for _ in range(limit):
        if not sched.has_work:
            return done
        plan = sched.plan()
        done.extend(plan.failed)
        if plan.entries:
            done.extend(sched.complete(plan, runner.run(plan)))
    raise AssertionError("the scheduler did not finish")


def expected(r):
    seq, out = list(r.prompt), []
    for _ in range(r.params.max_new_tokens):
        t = next_token(seq)
        if t in r.stop_set:
            break
        out.append(t)
        seq.append(t)
    return out


def test_prompts_are_cut_under_the_budget_first_come_first_served():
    cache, sched, runner = make(budget=16)
    for rid, n in enumerate((5, 17, 40)):
        sched.add(req(rid, n, max_new=2))
    plan = sched.plan()
    assert [(e.request.request_id, e.start, e.count, e.want_last) for e in plan.entries] == [(0, 0, 5, True), (1, 0, 11, False)]
    sched.complete(plan, runner.run(plan))
    plan = sched.plan()
    # the decode of request 0 first, then the rest of prompt 1, then the start of prompt 2
    assert [(e.request.request_id, e.start, e.count, e.want_last) for e in plan.entries] == \
        [(0, 5, 1, True), (1, 11, 6, True), (2, 0, 9, False)]
    assert plan.num_tokens == 16


def test_everything_finishes_with_the_tokens_of_an_unbatched_run():
    cache, sched, runner = make(budget=16)
    reqs = [req(0, 5, 8), req(1, 17, 8), req(2, 40, 8)]
    for r in reqs:
        sched.add(r)
    done = drive(sched, runner)
    assert {r.request_id for r in done} == {0, 1, 2}
    for r in reqs:
        assert r.status == FINISHED and r.finish_reason == "length" and r.generated == expected(r)
    assert cache.free_pages() == {0: 64, 1: 64} and cache.state_slots.free_count == 4
    assert max(sum(c for _, _, c, _ in step) for step in runner.steps) <= 16


def test_stop_token_ends_a_request_and_is_not_reported():
    cache, sched, runner = make()
    r = req(0, 6, max_new=50)
    stop_at = expected(r)[3]
    r.stop_set = (stop_at,)
    sched.add(r)
    drive(sched, runner)
    assert r.finish_reason == "stop" and r.stop_token == stop_at and stop_at not in r.generated
    assert r.generated == expected(r)


def test_batch_limit_and_state_slots():
    cache, sched, runner = make(max_batch=2, budget=64)
    for rid in range(5):
        sched.add(req(rid, 3, max_new=3))
    plan = sched.plan()
    assert [e.request.request_id for e in plan.entries] == [0, 1] and len(sched.waiting) == 3
    sched.complete(plan, runner.run(plan))
    done = drive(sched, runner)
    assert len(done) == 5 and all(len(step) <= 2 for step in runner.steps)


def test_pages_run_out_the_newest_is_preempted_and_recomputed():
    # 6 pages of 4 positions per group; two requests that grow to 14 positions each need 8 pages.
    cache, sched, runner = make(num_pages=6, page_size=4, budget=32, chunk=64)
    a, b = req(0, 6, max_new=8), req(1, 6, max_new=8)
    sched.add(a)
    sched.add(b)
    drive(sched, runner)
    assert sched.num_preemptions >= 1 and b.preemptions >= 1 and a.preemptions == 0
    assert a.generated == expected(a) and b.generated == expected(b)
    assert a.finish_reason == b.finish_reason == "length"
    # the preempted request came back through a prefill of prompt + what it had generated
    assert any(rid == 1 and start == 0 and count > 6 for step in runner.steps for rid, start, count, _ in step)
    assert cache.free_pages() == {0: 6, 1: 6}


def test_a_request_that_cannot_fit_alone_fails_and_the_others_go_on():
    cache, sched, runner = make(num_pages=3, page_size=4, budget=8, chunk=64)
    big, small = req(0, 30, max_new=2), req(1, 4, max_new=2)
    sched.add(big)
    sched.add(small)
    drive(sched, runner)
    assert big.finish_reason == "cache_full" and big.status == FINISHED
    assert small.finish_reason == "length" and small.generated == expected(small)
    assert cache.free_pages() == {0: 3, 1: 3} and not cache.requests


def test_chunked_group_alone_does_not_need_more_pages_than_a_chunk():
    # full layers would overflow; with only the chunked group (nope=()) a long prompt streams through
    from fakes import fake_blocks
    from sharpinference_b200.cache import CacheManager
    from sharpinference_b200.models.model import ScheduleEntry
    from sharpinference_b200.parts.base import CacheSpec
    import torch
    blocks = fake_blocks([CacheSpec("chunk", 8, 1, 8)])
    cache = CacheManager([ScheduleEntry(0)], blocks, page_size=4, num_pages=5, max_requests=2, dtype=torch.float32,
                         device="cpu", allocate=False)
    sched, runner = Scheduler(cache, max_batch=2, max_tokens_per_step=8), FakeRunner(cache)
    r = req(0, 100, max_new=5)
    sched.add(r)
    drive(sched, runner)
    assert r.finish_reason == "length" and r.generated == expected(r) and sched.num_preemptions == 0


def test_abort_frees_everything():
    cache, sched, runner = make()
    sched.add(req(0, 10, max_new=50))
    sched.add(req(1, 10, max_new=50))
    plan = sched.plan()
    sched.complete(plan, runner.run(plan))
    assert sched.abort(0).finish_reason == "abort"
    assert 0 not in cache.requests and 1 in cache.requests
    sched.abort(1)
    assert cache.free_pages() == {0: 64, 1: 64} and not sched.has_work
    assert sched.abort(99) is None


@pytest.mark.parametrize("seed", range(5))
def test_random_arrivals_with_few_pages(seed):
    rng = random.Random(seed)
    cache, sched, runner = make(num_pages=12, page_size=4, max_batch=4, budget=rng.choice([5, 9, 16]), chunk=8)
    reqs = [req(i, rng.choice([1, 2, 5, 9, 17, 23]), max_new=rng.choice([1, 3, 6])) for i in range(12)]
    pending = list(reqs)
    for _ in range(5000):
        if pending and rng.random() < 0.3:
            sched.add(pending.pop(0))
        if sched.has_work:
            plan = sched.plan()
            if plan.entries:
                sched.complete(plan, runner.run(plan))
        elif not pending:
            break
    for r in reqs:
        assert r.status == FINISHED
        if r.finish_reason == "length":
            assert r.generated == expected(r)
        else:
            assert r.finish_reason == "cache_full"
    assert cache.free_pages() == {0: 12, 1: 12}


def test_more_decodes_than_the_budget_take_turns():
    """Four requests decode under a budget of three tokens a step: nobody starves, the one left out changes
    from step to step, and pages are taken only for the decodes that run."""
    cache, sched, runner = make(num_pages=64, max_batch=4, budget=8)
    reqs = [req(i, 2, max_new=6) for i in range(4)]
    for r in reqs:
        sched.add(r)
    plan = sched.plan()                                   # all four prompts in one step
    sched.complete(plan, runner.run(plan))
    sched.max_tokens_per_step = 3
    left_out = []
    for _ in range(200):
        if not sched.has_work:
            break
        plan = sched.plan()
        assert plan.num_tokens <= 3
        deco = [r for r in sched.running if r.pending == 1 and r.computed >= len(r.prompt)]
        if len(deco) == 4:
            ran = {e.request.request_id for e in plan.entries}
            assert len(ran) == 3
            left_out.append(({0, 1, 2, 3} - ran).pop())
        free_before = dict(cache.free_pages())
        sched.complete(plan, runner.run(plan))
        # no page was counted for a request that did not run
        need = {0: 0, 1: 0}
        assert all(free_before[g] - cache.free_pages()[g] <= len(plan.entries) for g in need)
    assert not sched.has_work
    assert len(set(left_out)) == 4, f"the same requests were left out every time: {left_out}"
    assert all(a != b for a, b in zip(left_out, left_out[1:]))
    for r in reqs:
        assert r.finish_reason == "length" and r.generated == expected(r)


def test_a_plan_that_preempted_admits_nobody():
    # two requests fill the pool; when the newer one is sent back it must not return in the same plan
    cache, sched, runner = make(num_pages=4, page_size=4, budget=32, chunk=64)
    a, b = req(0, 7, max_new=8), req(1, 7, max_new=8)
    sched.add(a)
    sched.add(b)
    saw = False
    for _ in range(200):
        if not sched.has_work:
            break
        plan = sched.plan()
        if plan.preempted:
            saw = True
            assert all(e.request not in plan.preempted for e in plan.entries)
            assert all(r.status == WAITING for r in plan.preempted)
        if plan.entries:
            sched.complete(plan, runner.run(plan))
    assert saw and a.generated == expected(a) and b.generated == expected(b)
    assert cache.free_pages() == {0: 4, 1: 4}


def test_fail_and_fail_all_give_everything_back():
    cache, sched, runner = make()
    reqs = [req(i, 10, max_new=50) for i in range(6)]          # four run, two wait
    for r in reqs:
        sched.add(r)
    plan = sched.plan()
    sched.complete(plan, runner.run(plan))
    sched.fail(reqs[1], "broken")
    assert reqs[1].status == FINISHED and reqs[1].finish_reason == "error" and reqs[1].error == "broken"
    assert 1 not in cache.requests
    failed = sched.fail_all("the pass died")
    assert {r.request_id for r in failed} == {0, 2, 3, 4, 5}
    assert all(r.finish_reason == "error" and r.error == "the pass died" for r in failed)
    assert not sched.has_work and cache.free_pages() == {0: 64, 1: 64} and cache.state_slots.free_count == 4
    cache.check_invariants()
    sched.fail(reqs[0], "again")                                 # ending twice changes nothing
    assert reqs[0].error == "the pass died"
