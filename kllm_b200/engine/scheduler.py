"""Continuous batching above the step function.

Each ``step()`` forms one batch from whatever requests are live: one token for
every request that is decoding, then portions of prompts under what is left of
the token budget, admitting queued requests first-come-first-served while batch
slots, budget and pages last.  After the step each finished portion's last logits
are sampled; a request ends on an EOS id (the EOS token is emitted) or after
``max_new`` tokens and its pages are free for the next step at once.  This is the
loop of the reference's scheduler (engine/scheduler.go:95-237) with three
differences that the reference names as future work or cannot do:

* a prompt may be cut into portions over several steps (the reference admits a
  prompt only whole, :160-176, and rejects one longer than the budget, :67-70);
* a reservation is all-or-nothing, so a request that waits holds no half-filled
  table (the reference's waiting requests keep partial pages, :177-181);
* when pages run out for a request that is decoding, the youngest live request
  that is not yet part of the batch is preempted: its pages are given back and it
  returns to the head of the queue, to be recomputed from its tokens (prompt and
  what it generated).  ``on_pages_out="fail"`` keeps the reference's rule instead:
  that request alone fails with "kv reservation failed mid-stream" (:182).

The decisions are made by ``plan()`` on host data alone (requests, the cache
manager's counters), so they are tested without a GPU against a fake executor.

With an engine the loop is pipelined: a step is launched before the tokens of the step
before it have been read.  What a decoding request feeds into that step is then not a
token id from the host but "whatever was sampled for this request slot", which the
sampling kernel left on the device (``StepEntry.deferred``); positions, block tables
and the sampler's counters do not depend on the token.  The host reads a step's tokens
one step late, while the GPU already runs the next step, so its bookkeeping costs no
GPU time.  Consequences: a request that ends on an EOS id has one more step in
flight, whose token is thrown away (a request that ends on its count does not: that is
known in advance); and before anything is preempted, or when nothing can be planned,
everything in flight is collected first, so those decisions see complete requests.
``pipelined=False`` gives the plain loop (launch, read, book-keep), which is also what
the tests' fake executors get.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Any, Callable, Deque, List, Optional, Sequence, Tuple

from ..cache.manager import CacheManager, RequestCache
from .step import StepEntry

PENDING = -1     # stands in a request's tokens for one that was sampled but not read yet


class _NeedDrain(Exception):
    """Planning wants to preempt while steps are in flight: collect them first."""


@dataclass
class Request:
    rid: int
    prompt: List[int]
    max_new: int
    temperature: float = 0.0
    seed: int = 0
    tokens: List[int] = field(default_factory=list)     # prompt + generated so far
    generated: List[int] = field(default_factory=list)
    cache: Optional[RequestCache] = None
    fed: int = 0                  # how many of ``tokens`` are in the cache
    status: str = "waiting"       # waiting | running | finished | failed
    error: Optional[str] = None
    preemptions: int = 0
    sampled: int = 0              # tokens drawn for it so far, those not read yet included
    no_more: bool = False         # its last token (by count) is in flight: nothing more to plan

    @property
    def remaining(self) -> int:
        return len(self.tokens) - self.fed

    @property
    def done(self) -> bool:
        return self.status in ("finished", "failed")


@dataclass
class Metrics:
    steps: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    generated_tokens: int = 0
    preemptions: int = 0
    finished: int = 0
    failed: int = 0
    max_batch_seen: int = 0
    pages_high_water: int = 0


@dataclass
class PlannedEntry:
    request: Request
    n_tokens: int
    wants_logits: bool


@dataclass
class _InFlight:
    """A launched step whose tokens the host has not read."""
    rows: List[Tuple[Request, int]]     # per sampled row: the request and where in its tokens the result goes
    result: Any                         # what ``launch`` returned: ``result.tokens()`` waits and gives the list


class _EngineResult:
    """Sampled ids on their way to pinned host memory."""

    def __init__(self, pinned, event):
        self.pinned, self.event = pinned, event

    def tokens(self) -> List[int]:
        self.event.synchronize()
        return self.pinned.tolist()


class Scheduler:
    def __init__(self, engine=None, *, cache: Optional[CacheManager] = None,
                 execute: Optional[Callable] = None, max_batch: Optional[int] = None,
                 max_step_tokens: Optional[int] = None, max_seq: Optional[int] = None,
                 eos_token_ids: Sequence[int] = (), on_pages_out: str = "preempt",
                 pipelined: Optional[bool] = None, launch: Optional[Callable] = None):
        """With an ``Engine`` everything is taken from it.  Tests pass ``cache`` (a
        CacheManager, possibly without device memory) and either ``execute(entries,
        requests) -> list of next tokens`` for the entries that want logits (plain loop)
        or ``launch(entries, requests, keys) -> result`` whose ``result.tokens()`` gives
        that list later (pipelined loop; ``keys`` are the sampler's (seed, request id,
        index) per wanting entry, and a ``deferred`` entry's token is a placeholder for
        what the step before sampled for that request)."""
        if on_pages_out not in ("preempt", "fail"):
            raise ValueError("on_pages_out is 'preempt' or 'fail'")
        self.engine = engine
        if pipelined is None:
            pipelined = launch is not None or (engine is not None and execute is None)
        self.pipelined = bool(pipelined)
        if self.pipelined and launch is None:
            if engine is None or execute is not None:
                raise ValueError("the pipelined loop needs an engine or a launch function")
            launch = self._launch_on_engine
        self.launch = launch
        self._inflight: Deque[_InFlight] = deque()
        if engine is not None:
            cache = engine.cache
            execute = execute or self._execute_on_engine
            max_batch = max_batch or engine.options.max_batch
            max_step_tokens = max_step_tokens or engine.options.max_step_tokens
            max_seq = max_seq or engine.max_seq
            eos_token_ids = eos_token_ids or engine.eos_token_ids
        self.cache = cache
        self.execute = execute
        self.max_batch = min(int(max_batch), cache.max_requests)
        self.max_step_tokens = int(max_step_tokens)
        self.max_seq = int(max_seq)
        self.eos = set(int(e) for e in eos_token_ids)
        self.on_pages_out = on_pages_out
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.metrics = Metrics()
        self._next_rid = 0

    # ---- submission ------------------------------------------------------
    def submit(self, prompt: Sequence[int], max_new: int, temperature: float = 0.0, seed: int = 0) -> Request:
        prompt = [int(t) for t in prompt]
        if not prompt or max_new <= 0:
            raise ValueError("scheduler: empty prompt or non-positive max_new")   # scheduler.go:64-66
        total = len(prompt) + max_new
        if total > self.max_seq:
            raise ValueError(f"scheduler: prompt of {len(prompt)} tokens plus {max_new} new ones exceeds "
                             f"the sequence limit {self.max_seq}")
        # can it ever fit?  Asked of the cache manager group by group: a window group
        # needs only its window's pages however long the request is
        for g, pages in zip(self.cache.groups, self.cache.pages_ever_needed(total)):
            if pages > g.pool.n:
                raise ValueError(f"scheduler: the request needs {pages} pages of cache group {g.index}, "
                                 f"its pool has {g.pool.n}")
        r = Request(rid=self._next_rid, prompt=prompt, max_new=int(max_new),
                    temperature=float(temperature), seed=int(seed), tokens=list(prompt))
        self._next_rid += 1
        self.waiting.append(r)
        return r

    # ---- planning ----------------------------------------------------------
    def _preempt(self, r: Request) -> None:
        self.cache.close(r.cache)
        r.cache = None
        r.fed = 0
        r.status = "waiting"
        r.preemptions += 1
        self.running.remove(r)
        self.waiting.appendleft(r)
        self.metrics.preemptions += 1

    def _fail(self, r: Request, why: str) -> None:
        if r.cache is not None:
            self.cache.close(r.cache)
            r.cache = None
        r.status = "failed"
        r.error = why
        if r in self.running:
            self.running.remove(r)
        self.metrics.failed += 1

    def plan(self) -> List[PlannedEntry]:
        """Decide this step's batch.  May preempt or fail requests (pages run out)
        and admits from the queue; reserves nothing."""
        while True:
            entries = self._plan_once()
            if entries or not self.running:
                return entries
            # live requests but nothing can move: every one waits for pages that the
            # others hold.  The youngest gives way.
            if self._inflight:
                raise _NeedDrain()
            self._preempt(self.running[-1])

    def _plan_once(self) -> List[PlannedEntry]:
        budget = self.max_step_tokens
        planned_pages = [0] * len(self.cache.groups)
        entries: List[PlannedEntry] = []
        planned = set()

        def fits(r: Request, n: int) -> bool:
            need = self.cache.pages_for(r.cache, n)
            return all(planned_pages[i] + need[i] <= g.pool.free_count
                       for i, g in enumerate(self.cache.groups))

        def take(r: Request, n: int) -> None:
            nonlocal budget
            for i, c in enumerate(self.cache.pages_for(r.cache, n)):
                planned_pages[i] += c
            budget -= n
            entries.append(PlannedEntry(r, n, wants_logits=(n == r.remaining)))
            planned.add(r.rid)

        # 1. one token for every request that is decoding, oldest first
        for r in list(self.running):
            if r.remaining != 1 or r.status != "running" or r.no_more:
                continue
            if budget <= 0:
                break
            while not fits(r, 1):
                if self._inflight:
                    raise _NeedDrain()
                if self.on_pages_out == "fail":
                    self._fail(r, "kv reservation failed mid-stream: out of pages")
                    break
                victims = [v for v in self.running if v.rid not in planned and v is not r]
                victim = victims[-1] if victims else r
                self._preempt(victim)
                if victim is r:
                    break
            if r.status == "running":
                take(r, 1)
        # 2. portions for requests in the middle of a prompt, oldest first
        for r in list(self.running):
            if r.remaining <= 1 or budget <= 0:
                continue
            n = min(r.remaining, budget, self.cache.room_for(r.cache, planned_pages))
            if n > 0:
                take(r, n)
        # 3. admit from the queue in order, while slots, budget and pages last
        while self.waiting and len(self.running) < self.max_batch and budget > 0:
            r = self.waiting[0]
            r.cache = self.cache.open()
            n = min(r.remaining, budget, self.cache.room_for(r.cache, planned_pages))
            if n <= 0:
                self.cache.close(r.cache)
                r.cache = None
                break
            self.waiting.popleft()
            r.status = "running"
            self.running.append(r)
            take(r, n)
        return entries

    # ---- execution ---------------------------------------------------------
    def _execute_on_engine(self, entries: List[StepEntry], requests: List[Request]) -> List[int]:
        eng = self.engine
        logits = eng.runner.run(entries)
        if logits is None:
            return []
        wanting = [r for r, e in zip(requests, entries) if e.want]
        temps = [r.temperature for r in wanting]
        keys = [(r.seed, r.rid, len(r.generated)) for r in wanting]
        return eng.sampler.sample(logits, temps, keys).tolist()

    # ---- the pipelined loop ----------------------------------------------------
    def _launch_on_engine(self, entries: List[StepEntry], requests: List[Request], keys):
        import torch
        eng = self.engine
        logits = eng.runner.run(entries)
        if logits is None:
            return None
        wanting = [r for r, e in zip(requests, entries) if e.want]
        if len(wanting) == len(requests):
            slots = eng.runner.last_ctx.state_slots
        else:
            slots = torch.tensor([r.cache.state_slot for r in wanting], dtype=torch.int32).to(
                logits.device, non_blocking=True)
        # the sampling kernel writes its choices into pinned host memory itself: no copy after it
        pinned = torch.empty(len(wanting), dtype=torch.int32, pin_memory=True)
        eng.sampler.sample(logits, [r.temperature for r in wanting], keys,
                           last_token=eng.runner.last_token, slots=slots, host_out=pinned)
        event = torch.cuda.Event()
        event.record()
        return _EngineResult(pinned, event)

    def _launch(self, plan: List[PlannedEntry]) -> None:
        entries, requests = [], []
        for p in plan:
            r = p.request
            toks = r.tokens[r.fed:r.fed + p.n_tokens]
            entries.append(StepEntry(r.cache, toks, [p.n_tokens - 1] if p.wants_logits else [],
                                     deferred=(p.n_tokens == 1 and toks[0] == PENDING)))
            requests.append(r)
        keys = [(r.seed, r.rid, r.sampled) for r, e in zip(requests, entries) if e.want]
        try:
            result = self.launch(entries, requests, keys)
        except Exception as e:  # a failed step fails its requests (scheduler.go:197-203)
            for r in requests:
                if r.cache is not None and not r.cache.closed:
                    self.cache.trim_reservation(r.cache)
                self._fail(r, f"step failed: {e}")
            raise
        self.metrics.steps += 1
        self.metrics.max_batch_seen = max(self.metrics.max_batch_seen, len(plan))
        self.metrics.pages_high_water = max([self.metrics.pages_high_water] +
                                            [g.pool.high_water for g in self.cache.groups])
        rows: List[Tuple[Request, int]] = []
        for p in plan:
            r = p.request
            if p.n_tokens == 1 and r.fed >= len(r.prompt):
                self.metrics.decode_tokens += 1
            else:
                self.metrics.prefill_tokens += p.n_tokens
            r.fed += p.n_tokens
            if p.wants_logits:
                r.tokens.append(PENDING)
                rows.append((r, len(r.tokens) - 1))
                r.sampled += 1
                r.no_more = r.sampled >= r.max_new
        if rows:
            self._inflight.append(_InFlight(rows, result))

    def _collect(self, rec: _InFlight) -> List[Tuple[Request, int]]:
        events: List[Tuple[Request, int]] = []
        for (r, idx), tok in zip(rec.rows, rec.result.tokens()):
            if r.status != "running":        # ended on an EOS id a step earlier: this token is not its
                continue
            r.tokens[idx] = tok
            r.generated.append(tok)
            self.metrics.generated_tokens += 1
            events.append((r, tok))
            if tok in self.eos or len(r.generated) >= r.max_new:
                del r.tokens[idx + 1:]       # the placeholder of a step launched since
                self.cache.close(r.cache)    # a step in flight that still reads these pages runs before
                r.cache = None               # any later step that could be given them (one stream)
                r.status = "finished"
                self.running.remove(r)
                self.metrics.finished += 1
        return events

    def _collect_all(self) -> List[Tuple[Request, int]]:
        events: List[Tuple[Request, int]] = []
        while self._inflight:
            events += self._collect(self._inflight.popleft())
        return events

    def _step_pipelined(self) -> List[Tuple[Request, int]]:
        events: List[Tuple[Request, int]] = []
        try:
            plan = self.plan()
        except _NeedDrain:
            events += self._collect_all()
            plan = self.plan()
        if plan:
            self._launch(plan)
        # the step just launched stays in flight; everything before it is read now,
        # while the GPU works on it
        keep = 1 if plan else 0
        while len(self._inflight) > keep:
            events += self._collect(self._inflight.popleft())
        return events

    def step(self) -> List[Tuple[Request, int]]:
        """Run one batch; returns (request, new token) for every token that became known
        (pipelined: the tokens of the step before the one that this call launches)."""
        if self.pipelined:
            return self._step_pipelined()
        plan = self.plan()
        if not plan:
            return []
        entries, requests = [], []
        for p in plan:
            r = p.request
            toks = r.tokens[r.fed:r.fed + p.n_tokens]
            entries.append(StepEntry(r.cache, toks, [p.n_tokens - 1] if p.wants_logits else []))
            requests.append(r)
        try:
            new_tokens = self.execute(entries, requests)
        except Exception as e:  # a failed step fails its requests (scheduler.go:197-203)
            for r in requests:
                if r.cache is not None and not r.cache.closed:
                    self.cache.trim_reservation(r.cache)
                self._fail(r, f"step failed: {e}")
            raise
        self.metrics.steps += 1
        self.metrics.max_batch_seen = max(self.metrics.max_batch_seen, len(plan))
        self.metrics.pages_high_water = max([self.metrics.pages_high_water] +
                                            [g.pool.high_water for g in self.cache.groups])
        events: List[Tuple[Request, int]] = []
        it = iter(new_tokens)
        for p in plan:
            r = p.request
            if p.n_tokens == 1 and r.fed >= len(r.prompt):
                self.metrics.decode_tokens += 1
            else:
                self.metrics.prefill_tokens += p.n_tokens
            r.fed += p.n_tokens
            if not p.wants_logits:
                continue
            tok = int(next(it))
            r.tokens.append(tok)
            r.generated.append(tok)
            self.metrics.generated_tokens += 1
            events.append((r, tok))
            if tok in self.eos or len(r.generated) >= r.max_new:
                self.cache.close(r.cache)
                r.cache = None
                r.status = "finished"
                self.running.remove(r)
                self.metrics.finished += 1
        return events

    def run(self, max_steps: int = 1 << 30) -> None:
        """Step until every submitted request has ended."""
        steps = 0
        while (self.waiting or self.running or self._inflight) and steps < max_steps:
            before = (len(self.waiting), len(self.running), self.metrics.steps)
            self.step()
            steps += 1
            if ((len(self.waiting), len(self.running), self.metrics.steps) == before and not self.running
                    and not self._inflight and self.waiting):
                # nothing live, nothing admitted: the head of the queue can never fit
                r = self.waiting.popleft()
                self._fail(r, "request cannot be admitted: no pages")

    def stop(self) -> None:
        """Fail everything in flight (scheduler.go:130-134)."""
        self._inflight.clear()
        for r in list(self.running) + list(self.waiting):
            self._fail(r, "scheduler stopped")
        self.waiting.clear()
