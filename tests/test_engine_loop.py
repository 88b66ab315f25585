"""The request loop of the engine with stand-ins for the step function and the sampler (no GPU): what happens
when a step cannot run.  Faults are made on the host only: a step function that raises, a request with a
token outside the vocabulary, a page pool that reports exhaustion although the plan counted otherwise."""
import zlib
from types import SimpleNamespace

import pytest

from fakes import llama_like_manager
from sharpinference_b200.cache import OutOfPages
from sharpinference_b200.engine import Engine, EngineOptions, StepError
from sharpinference_b200.sampling import SamplingParams

VOCAB = 100


def next_token(tokens):
    return zlib.crc32(bytes(str(list(tokens)), "ascii")) % 90 + 3


class FakeStep:
    """Reserves and commits like the step function; its 'logits' are the next token of every wanted row.
    ``fail_on`` = set of step numbers (counted over calls) on which it raises after the pages were reserved."""

    def __init__(self, cache, fail_on=(), error=RuntimeError("injected: the device pass failed")):
        self.cache, self.fail_on, self.error = cache, set(fail_on), error
        self.calls = 0
        self.history = {}
        self.graph_replays = 0
        self.resets = 0

    def run(self, entries):
        for e in entries:
            for t in e.tokens:
                if not 0 <= t < VOCAB:
                    raise StepError(f"request {e.request_id!r}: token id {t} is outside the vocabulary", e.request_id)
        self.cache.reserve([(e.request_id, len(e.tokens)) for e in entries])
        call, self.calls = self.calls, self.calls + 1
        if call in self.fail_on:
            raise self.error
        out = []
        for e in entries:
            seq = self.history.setdefault(e.request_id, [])
            if self.cache.get(e.request_id).length == 0:
                seq.clear()                          # a request that was sent back starts over
            assert self.cache.get(e.request_id).length == len(seq)
            seq.extend(e.tokens)
            self.cache.commit(e.request_id, len(e.tokens))
            out.extend(next_token(seq[:len(seq) - len(e.tokens) + w + 1]) for w in e.want)
        return out

    def flush_status(self):
        pass

    def reset_after_failure(self):
        self.resets += 1
        self.history.clear()


class FakeSampler:
    def sample(self, logits, states):
        assert len(logits) == len(states)
        return list(logits)


def make_engine(num_pages=64, page_size=4, max_batch=4, budget=16, chunk=8, **step_args):
    cache = llama_like_manager(num_pages=num_pages, page_size=page_size, chunk=chunk, max_requests=max_batch)
    model = SimpleNamespace(vocab_size=VOCAB, eos_token_ids=(), act_dtype=None)
    runner = FakeStep(cache, **step_args)
    eng = Engine.from_parts(model=model, cache=cache, runner=runner, sampler=FakeSampler(),
                            options=EngineOptions(page_size=page_size, max_batch=max_batch, max_tokens_per_step=budget))
    return eng, cache, runner


def prompt(i, n):
    return [((i + 1) * 7 + j) % 90 + 3 for j in range(n)]


def expected(p, n):
    seq, out = list(p), []
    for _ in range(n):
        out.append(next_token(seq))
        seq.append(out[-1])
    return out


GREEDY = SamplingParams(temperature=0.0, max_new_tokens=5)


def all_free(cache, pages):
    cache.check_invariants()
    return cache.free_pages() == {0: pages, 1: pages} and not cache.requests and \
        cache.state_slots.free_count == cache.max_requests


def test_generate_with_stand_ins():
    eng, cache, _ = make_engine()
    prompts = [prompt(i, n) for i, n in enumerate((5, 17, 40))]
    assert eng.generate(prompts, GREEDY) == [expected(p, 5) for p in prompts]
    assert all_free(cache, 64) and not eng._requests


@pytest.mark.parametrize("k", [0, 1, 3, 6])
def test_a_step_that_raises_ends_every_request_with_the_error_and_the_engine_goes_on(k):
    eng, cache, runner = make_engine(fail_on={k})
    ids = [eng.add_request(prompt(i, n), GREEDY) for i, n in enumerate((5, 17, 40, 9, 3))]   # one more than the batch
    reported = {}
    while eng.has_unfinished:
        for out in eng.step():
            reported[out.request_id] = out
    assert set(reported) == set(ids)
    failed = [o for o in reported.values() if o.finish_reason == "error"]
    assert failed and all("injected" in o.error and o.finished for o in failed)
    # whoever finished before the failing step has its tokens; nobody is left half-way
    for o in reported.values():
        if o.finish_reason == "length":
            assert o.tokens == expected(o.prompt, 5)
    assert isinstance(eng.last_error, RuntimeError) and eng.stats["failed_steps"] == 1 and runner.resets == 1
    assert all_free(cache, 64) and not eng.has_unfinished and not eng._requests
    # the same engine serves new requests
    p = prompt(9, 11)
    assert eng.generate([p], GREEDY) == [expected(p, 5)]
    assert all_free(cache, 64)


def test_generate_raises_when_its_requests_failed():
    eng, cache, _ = make_engine(fail_on={1})
    with pytest.raises(RuntimeError, match="injected"):
        eng.generate([prompt(0, 30), prompt(1, 4)], GREEDY)
    assert all_free(cache, 64)
    assert eng.generate([prompt(2, 6)], GREEDY) == [expected(prompt(2, 6), 5)]


def test_a_bad_token_ends_its_request_alone():
    eng, cache, runner = make_engine()
    good = [prompt(0, 6), prompt(1, 20)]
    a = eng.add_request(good[0], GREEDY)
    eng.model.vocab_size = 10 ** 6                   # let the bad id past add_request: the step function finds it
    bad = eng.add_request([5, 6, VOCAB + 7, 8], GREEDY)
    eng.model.vocab_size = VOCAB
    b = eng.add_request(good[1], GREEDY)
    reported = {}
    while eng.has_unfinished:
        for out in eng.step():
            reported[out.request_id] = out
    assert reported[bad].finish_reason == "error" and "outside the vocabulary" in reported[bad].error
    assert reported[a].tokens == expected(good[0], 5) and reported[b].tokens == expected(good[1], 5)
    assert eng.last_error is None and eng.stats["failed_steps"] == 0 and runner.resets == 0
    assert all_free(cache, 64)


def test_a_pool_that_reports_exhaustion_mid_plan():
    """The plan counted on pages that the pool then refuses (all or nothing: none is taken).  The newest
    running request goes back to the queue, the step is planned again, and everything still finishes."""
    eng, cache, runner = make_engine(num_pages=16)
    inner, calls = cache.reserve, {"n": 0}

    def flaky(wants):
        calls["n"] += 1
        if calls["n"] in (2, 5):
            raise OutOfPages(0, 99, 0)
        return inner(wants)

    cache.reserve = flaky
    prompts = [prompt(i, n) for i, n in enumerate((6, 9, 5))]
    assert eng.generate(prompts, GREEDY) == [expected(p, 5) for p in prompts]
    assert eng.stats["preemptions"] >= 2 and eng.stats["failed_steps"] == 0
    assert all_free(cache, 16)


def test_exhaustion_with_one_request_ends_it_cache_full():
    eng, cache, runner = make_engine(num_pages=16)
    cache.reserve = lambda wants: (_ for _ in ()).throw(OutOfPages(0, 99, 0))
    rid = eng.add_request(prompt(0, 6), GREEDY)
    outs = []
    while eng.has_unfinished:
        outs.extend(eng.step())
    assert [o.finish_reason for o in outs] == ["cache_full"] and outs[0].request_id == rid
    assert all_free(cache, 16)


def test_finished_requests_are_not_kept_for_ever():
    eng, cache, _ = make_engine()
    eng.options.keep_finished = 3
    ids = []
    for i in range(8):
        ids.append(eng.add_request(prompt(i, 4), SamplingParams(temperature=0.0, max_new_tokens=2)))
        while eng.has_unfinished:
            eng.step()
    assert not eng._requests and list(eng._finished) == ids[-3:]
    assert eng.output(ids[-1]).tokens == expected(prompt(7, 4), 2)
    with pytest.raises(KeyError):
        eng.output(ids[0])
    assert eng.metrics()["tracked_requests"] == 0


def test_abort_reports_and_forgets():
    eng, cache, _ = make_engine()
    a = eng.add_request(prompt(0, 30), GREEDY)
    b = eng.add_request(prompt(1, 5), GREEDY)
    eng.step()
    out = eng.abort(a)                       # in the middle of its prompt (30 tokens, budget 16)
    assert out.finish_reason == "abort" and out.finished and a not in eng._requests
    while eng.has_unfinished:
        eng.step()
    assert eng.output(b).tokens == expected(prompt(1, 5), 5) and all_free(cache, 64)
    assert eng.abort("nobody") is None
