"""The scheduler's decisions, on the host: a fake executor stands for the GPU and
answers with a token that depends only on the request's tokens so far, so every
way of batching, cutting and preempting must give the tokens of a solo run."""
import random

import pytest

from kllm_b200.cache import CacheManager
from kllm_b200.engine.scheduler import Scheduler
from kllm_b200.parts.spec import PagedKVNeed

NEED = [PagedKVNeed(2, 16), PagedKVNeed(2, 16)]
EOS = 99


def next_token(tokens):
    h = 17
    for t in tokens:
        h = (h * 31 + t + 7) % 1009
    return h % 97          # never EOS unless a test plants it


class FakeExecutor:
    """Checks what a real step would check and reserves/commits like it."""

    def __init__(self, cache, budget, planted_eos=None):
        self.cache, self.budget, self.planted_eos = cache, budget, planted_eos or {}
        self.batches = []

    def __call__(self, entries, requests):
        assert sum(len(e.tokens) for e in entries) <= self.budget
        assert len({id(e.request) for e in entries}) == len(entries)
        assert self.cache.can_reserve_all([(e.request, len(e.tokens)) for e in entries])
        out = []
        self.batches.append([(r.rid, len(e.tokens), bool(e.want)) for e, r in zip(entries, requests)])
        for e, r in zip(entries, requests):
            assert list(e.tokens) == r.tokens[r.fed:r.fed + len(e.tokens)]
            assert e.request.length == r.fed
            self.cache.reserve(e.request, len(e.tokens))
            self.cache.commit(e.request, len(e.tokens))
            if e.want:
                assert list(e.want) == [len(e.tokens) - 1] and r.fed + len(e.tokens) == len(r.tokens)
                tok = next_token(r.tokens)
                if self.planted_eos.get(r.rid) == len(r.generated):
                    tok = EOS
                out.append(tok)
        self.cache.audit()
        return out


def make(num_pages=64, page_size=4, max_batch=4, budget=32, max_seq=256, on_pages_out="preempt", planted=None):
    cache = CacheManager(NEED, page_size, num_pages, max_requests=max_batch, allocate=False)
    ex = FakeExecutor(cache, budget, planted)
    s = Scheduler(cache=cache, execute=ex, max_batch=max_batch, max_step_tokens=budget, max_seq=max_seq,
                  eos_token_ids=[EOS], on_pages_out=on_pages_out)
    return s, ex, cache


def solo(prompt, max_new):
    toks, out = list(prompt), []
    for _ in range(max_new):
        out.append(next_token(toks))
        toks.append(out[-1])
    return out


def test_single_request_whole_prompt_then_decodes():
    s, ex, cache = make()
    r = s.submit([1, 2, 3, 4, 5], 4)
    s.run()
    assert r.status == "finished" and r.generated == solo([1, 2, 3, 4, 5], 4)
    assert ex.batches == [[(0, 5, True)], [(0, 1, True)], [(0, 1, True)], [(0, 1, True)]]
    assert cache.free_pages() == [64] and s.metrics.prefill_tokens == 5 and s.metrics.decode_tokens == 3


def test_prompt_is_cut_under_the_budget_and_decodes_go_first():
    s, ex, _ = make(budget=8)
    a = s.submit(list(range(3)), 6)
    s.step()                                   # a prefilled whole
    b = s.submit(list(range(20)), 2)           # 20 tokens under a budget of 8, one of them a's decode
    s.run()
    assert ex.batches[1] == [(0, 1, True), (1, 7, False)]
    assert ex.batches[2] == [(0, 1, True), (1, 7, False)]
    assert ex.batches[3] == [(0, 1, True), (1, 6, True)]
    assert a.generated == solo(list(range(3)), 6) and b.generated == solo(list(range(20)), 2)


def test_admission_is_fifo_and_bounded_by_slots():
    s, ex, _ = make(max_batch=2, budget=64)
    rs = [s.submit([i, i + 1], 3) for i in range(5)]
    s.step()
    assert [x[0] for x in ex.batches[0]] == [0, 1] and len(s.waiting) == 3
    s.run()
    assert all(r.generated == solo(r.prompt, 3) for r in rs)
    first_seen = {}
    for i, b in enumerate(ex.batches):
        for rid, _, _ in b:
            first_seen.setdefault(rid, i)
    assert [first_seen[i] for i in range(5)] == sorted(first_seen[i] for i in range(5))
    assert s.metrics.max_batch_seen == 2 and s.metrics.finished == 5


def test_eos_ends_a_request_and_is_emitted():
    s, ex, cache = make(planted={0: 2})
    r = s.submit([5, 6, 7], 10)
    other = s.submit([8], 4)
    s.run()
    assert r.generated[-1] == EOS and len(r.generated) == 3 and r.status == "finished"
    assert other.generated == solo([8], 4)
    assert cache.free_pages() == [64]


def test_submit_refuses_what_can_never_run():
    s, _, _ = make(num_pages=4, page_size=4, max_seq=64)
    with pytest.raises(ValueError):
        s.submit([], 3)
    with pytest.raises(ValueError):
        s.submit([1], 0)
    with pytest.raises(ValueError, match="sequence limit"):
        s.submit([1] * 60, 5)
    with pytest.raises(ValueError, match="pages"):
        s.submit([1] * 10, 8)           # 18 tokens need 5 pages of 4, the pool has 4


def test_pages_run_out_while_decoding_preempts_the_youngest():
    # 6 pages of 4 tokens; two requests of 8 prompt tokens fill 4 pages; both decode until
    # the pool is full, then the younger gives way, is recomputed later, and both end with
    # the tokens of a solo run
    s, ex, cache = make(num_pages=6, page_size=4, budget=32)
    a = s.submit(list(range(8)), 12)
    b = s.submit(list(range(50, 58)), 12)
    s.run()
    assert a.generated == solo(a.prompt, 12) and b.generated == solo(b.prompt, 12)
    assert s.metrics.preemptions >= 1 and b.preemptions >= 1 and a.preemptions == 0
    assert cache.free_pages() == [6]
    # the recomputation fed prompt and generated tokens in one portion
    assert any(n > 8 for batch in ex.batches for rid, n, _ in batch if rid == b.rid)


def test_pages_run_out_fail_mode_fails_that_request_alone():
    s, ex, cache = make(num_pages=6, page_size=4, budget=32, on_pages_out="fail")
    a = s.submit(list(range(8)), 12)
    b = s.submit(list(range(50, 58)), 12)
    s.run()
    failed = [r for r in (a, b) if r.status == "failed"]
    done = [r for r in (a, b) if r.status == "finished"]
    assert len(failed) == 1 and len(done) == 1
    assert "mid-stream" in failed[0].error
    assert done[0].generated == solo(done[0].prompt, 12)
    assert cache.free_pages() == [6]


def test_two_prompts_that_cannot_both_fit_do_not_block_each_other():
    # each needs 5 of 6 pages; the second waits holding nothing until the first has ended
    s, ex, cache = make(num_pages=6, page_size=4, budget=6)
    a = s.submit(list(range(17)), 2)
    b = s.submit(list(range(30, 47)), 2)
    s.run()
    assert a.generated == solo(a.prompt, 2) and b.generated == solo(b.prompt, 2)
    assert cache.free_pages() == [6]


def test_stop_fails_everything_in_flight():
    s, _, cache = make()
    a = s.submit([1, 2, 3], 5)
    s.step()
    b = s.submit([4], 5)
    s.stop()
    assert a.status == b.status == "failed" and a.error == "scheduler stopped"
    assert cache.free_pages() == [64]


def test_a_failing_step_fails_its_requests_and_frees_their_pages():
    s, ex, cache = make()

    def boom(entries, requests):
        raise RuntimeError("device fell over")

    a = s.submit([1, 2, 3], 5)
    s.execute = boom
    with pytest.raises(RuntimeError):
        s.step()
    assert a.status == "failed" and "device fell over" in a.error and cache.free_pages() == [64]


@pytest.mark.parametrize("seed", range(6))
def test_random_workloads_match_solo_runs(seed):
    rng = random.Random(seed)
    page = rng.choice([1, 4, 16])
    s, ex, cache = make(num_pages=rng.choice([24, 40, 200]) * 4 // page + 8, page_size=page,
                        max_batch=rng.choice([1, 2, 4]), budget=rng.choice([8, 24, 100]), max_seq=128)
    reqs = []
    for _ in range(12):
        prompt = [rng.randrange(90) for _ in range(rng.choice([1, 2, 5, 17, 40]))]
        reqs.append(s.submit(prompt, rng.choice([1, 3, 20])))
        for _ in range(rng.randrange(3)):
            s.step()
    s.run(max_steps=5000)
    for r in reqs:
        assert r.status == "finished" and r.generated == solo(r.prompt, r.max_new), r.rid
    assert cache.free_pages() == [g.pool.n for g in cache.groups]
    cache.audit()


# ---- the pipelined loop: a step is launched before the tokens of the step before are read ----

class FakeLauncher(FakeExecutor):
    """Like the GPU with the pipelined loop: it runs a step when it is launched, keeps
    what it sampled per request (the device's table of last tokens) and hands the host a
    result that is read later.  A deferred entry's token is a placeholder; the real one
    is what this launcher sampled for that request in its step before."""

    def __init__(self, cache, budget, planted_eos=None):
        super().__init__(cache, budget, planted_eos)
        self.real = {}            # request id -> every token as the device knows it

    def launch(self, entries, requests, keys):
        from kllm_b200.engine.scheduler import PENDING
        assert sum(len(e.tokens) for e in entries) <= self.budget
        assert self.cache.can_reserve_all([(e.request, len(e.tokens)) for e in entries])
        self.batches.append([(r.rid, len(e.tokens), bool(e.want)) for e, r in zip(entries, requests)])
        out, keys = [], list(keys)
        for e, r in zip(entries, requests):
            known = self.real.setdefault(r.rid, list(r.prompt))
            if r.fed == 0:                                   # a new or recomputed request: its tokens are on the host
                known[:] = [t for t in r.tokens if t != PENDING]
            toks = list(e.tokens)
            if e.deferred:
                assert toks == [PENDING] and len(known) == r.fed + 1
            else:
                assert PENDING not in toks and toks == known[r.fed:r.fed + len(toks)]
            assert e.request.length == r.fed
            self.cache.reserve(e.request, len(toks))
            self.cache.commit(e.request, len(toks))
            if e.want:
                seed, rid, index = keys.pop(0)
                assert rid == r.rid and index == len(known) - len(r.prompt)
                tok = EOS if self.planted_eos.get(r.rid) == index else next_token(known[:r.fed + len(toks)])
                known.append(tok)
                out.append(tok)
        self.cache.audit()

        class Result:
            def tokens(_):
                return out
        return Result()


def make_pipelined(num_pages=64, page_size=4, max_batch=4, budget=32, max_seq=256, planted=None):
    cache = CacheManager(NEED, page_size, num_pages, max_requests=max_batch, allocate=False)
    ex = FakeLauncher(cache, budget, planted)
    s = Scheduler(cache=cache, launch=ex.launch, max_batch=max_batch, max_step_tokens=budget, max_seq=max_seq,
                  eos_token_ids=[EOS])
    assert s.pipelined
    return s, ex, cache


def test_pipelined_loop_gives_the_solo_tokens_and_lags_one_step():
    s, ex, cache = make_pipelined()
    r = s.submit([1, 2, 3, 4, 5], 4)
    assert s.step() == []                      # launched, nothing read yet
    ev = s.step()                              # second step launched, first one read
    assert [t for _, t in ev] == solo([1, 2, 3, 4, 5], 1)
    s.run()
    assert r.status == "finished" and r.generated == solo([1, 2, 3, 4, 5], 4)
    # the count is known in advance: exactly four steps, no step for a fifth token
    assert ex.batches == [[(0, 5, True)], [(0, 1, True)], [(0, 1, True)], [(0, 1, True)]]
    assert cache.free_pages() == [64]


def test_pipelined_loop_drops_the_token_in_flight_after_an_eos():
    s, ex, cache = make_pipelined(planted={0: 2})
    a, b = s.submit([5, 6, 7], 10), s.submit([8, 9], 6)
    s.run()
    assert a.generated == solo([5, 6, 7], 2) + [EOS]
    assert b.generated == solo([8, 9], 6)
    # a's EOS was sampled in step 2 and read after step 3 was launched: a is in step 3, not in step 4
    assert [x[0] for x in ex.batches[3]] == [0, 1] and [x[0] for x in ex.batches[4]] == [1]
    assert a.tokens == [5, 6, 7] + a.generated and cache.free_pages() == [64]


@pytest.mark.parametrize("seed", range(8))
def test_pipelined_loop_under_random_load_and_few_pages(seed):
    """Random prompts, budgets and planted ends with so few pages that requests are
    preempted: before any preemption what is in flight is read, so every request still
    says what it says alone."""
    rng = random.Random(seed)
    planted = {i: rng.randrange(1, 8) for i in range(12) if rng.random() < 0.4}
    s, ex, cache = make_pipelined(num_pages=rng.choice([10, 14, 24]), page_size=4, max_batch=rng.choice([2, 3, 4]),
                                  budget=rng.choice([8, 16, 32]), max_seq=64, planted=planted)
    reqs = []
    for i in range(12):
        reqs.append(s.submit([rng.randrange(90) for _ in range(rng.randrange(1, 20))], rng.randrange(1, 12)))
        for _ in range(rng.randrange(0, 3)):
            s.step()
    s.run()
    for r in reqs:
        assert r.status == "finished"
        want = solo(r.prompt, r.max_new)
        if r.rid in planted and planted[r.rid] < r.max_new:
            want = want[:planted[r.rid]] + [EOS]
        assert r.generated == want, r.rid
    cache.audit()
    assert cache.free_pages() == [cache.num_pages] and not s._inflight


def test_admission_asks_each_group_what_a_request_can_ever_need():
    """A model whose layers all read a window of 6 keys: a request of 100 tokens fits a pool
    of 4 pages of 4 tokens (3 pages for the window's reach plus the page being written),
    although 100 tokens are 25 pages; a group that keeps every key still refuses it."""
    window = [PagedKVNeed(2, 16, window=6)]
    cache = CacheManager(window, 4, 4, max_requests=2, allocate=False)
    assert cache.pages_ever_needed(100) == [3] and cache.pages_ever_needed(5) == [2]
    ex = FakeExecutor(cache, 8)
    s = Scheduler(cache=cache, execute=ex, max_batch=2, max_step_tokens=8, max_seq=256, eos_token_ids=[EOS])
    prompt = [(7 * i) % 90 for i in range(60)]
    r = s.submit(prompt, 40)
    s.run()
    assert r.status == "finished" and r.generated == solo(prompt, 40)
    assert cache.free_pages() == [4] and max(n for b in ex.batches for _, n, _ in b) <= 8
    both = CacheManager(window + [PagedKVNeed(2, 16)], 4, 4, max_requests=2, allocate=False)
    assert both.pages_ever_needed(100) == [3, 25]
    s2 = Scheduler(cache=both, execute=FakeExecutor(both, 8), max_batch=2, max_step_tokens=8, max_seq=256)
    with pytest.raises(ValueError, match="25 pages of cache group 1"):
        s2.submit(prompt, 40)
    s2.submit(prompt[:10], 6)               # 16 tokens: 4 pages of the group that keeps every key
    s2.run()
    assert both.free_pages() == [4, 4]
