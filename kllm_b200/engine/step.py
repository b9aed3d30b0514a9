"""The step function: one batch of (request, its next tokens) through the model.

A batch may hold portions of prompts beside single decoded tokens, cut anywhere.
It runs only the tokens it is given, as one batch, against the cache that earlier
steps left, and returns float32 logits at the places that were asked for.  This
is the role of ``te_forward_batch`` (reference backend/model.cu:995-1195) with two
differences: logits come from the places the caller names (the reference returns
each request's last row, :1184-1188), and the per-step token budget is a knob of
its own (the reference ties it to the sequence cap, engine/engine.go:18).

Everything is validated on the host before anything is launched (as :1000-1043):
an invalid step changes neither the cache nor the device.  Pages are reserved for
all entries together or not at all, and committed after the launch.
"""
from __future__ import annotations

import gc

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager, OutOfPages, RequestCache
from ..parts.context import StepContext
from ..parts.model import DecoderModel


class StepError(ValueError):
    """The batch is not one this engine can run; nothing was changed."""


@dataclass
class StepEntry:
    request: RequestCache
    tokens: Sequence[int]
    want: Sequence[int] = ()      # places among ``tokens`` whose logits are wanted
    deferred: bool = False        # the one token is what the sampler chose for this request in the step
                                  # before; it is still on the device (``tokens`` holds a placeholder)


class GraphedDecode:
    """One decode step of a fixed batch size as a CUDA graph.

    A decode step of B requests launches over a hundred small kernels; replayed as
    one graph they cost one launch.  The graph reads the step's description (token
    ids, positions, block tables, state slots) from device buffers at fixed
    addresses that are refilled before every replay, and leaves the logits of all B
    tokens in a buffer of its own.  Launch shapes are fixed at capture: the block
    table is as wide as the longest sequence allows and the decode attention cuts
    every context as if it had that length.  The first step of a batch size runs
    eagerly on the same buffers (which also warms up every library), the capture
    follows without executing anything, and later steps replay.
    """

    def __init__(self, runner: "StepRunner", batch: int):
        self.runner = runner
        self.batch = batch
        cache, dev = runner.cache, runner.device
        self.width = max(1, -(-runner.max_seq // cache.page_size))
        B = batch
        sizes = [B, B, B, B + 1, B, B, B, B] + [B * self.width for _ in cache.groups]
        self.offs = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
        total = int(self.offs[-1])
        # two pinned staging buffers that take turns: the host may fill the next step's
        # while the copy of this step's has not run yet
        self.hosts = [torch.empty(total, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self.copied = [None, None]                  # event after the last copy out of each staging buffer
        self.turn = 0
        self.dev = torch.zeros(total, dtype=torch.int32, device=dev)
        o = self.offs
        for host in self.hosts:
            h = host.numpy()
            h[:] = 0
            h[o[2]:o[3]] = np.arange(B)             # token_req: token i belongs to request i
            h[o[3]:o[4]] = np.arange(B + 1)         # q_start
            h[o[7]:o[8]] = np.arange(B)             # every row is wanted
        part = lambda i: self.dev[int(o[i]):int(o[i + 1])]
        tables = {gi: part(8 + gi).view(B, self.width) for gi in range(len(cache.groups))}
        self.ctx = StepContext(
            n_tokens=B, n_requests=B, token_ids=part(0), positions=part(1), token_req=part(2), q_start=part(3),
            start_pos=part(4), ctx_len=part(5), state_slots=part(6), block_tables=tables, want_rows=part(7),
            n_want=B, host_n_new=[1] * B, host_start_pos=[0] * B, max_new=1, max_ctx=runner.max_seq,
            all_single=True, split_bound=runner.max_seq, last_token=runner.last_token)
        self.caches = cache.layer_caches(tables)
        self.graph = None
        self.logits = None
        self.launches = 0

    def fill(self, entries: Sequence["StepEntry"]) -> None:
        # a staging buffer is reused every other step: the copy that read it last must be over
        self.turn ^= 1
        host = self.hosts[self.turn]
        if self.copied[self.turn] is not None:
            self.copied[self.turn].synchronize()
        o, h, B, W = self.offs, host.numpy(), self.batch, self.width
        h[o[0]:o[1]] = [-(e.request.state_slot + 1) if e.deferred else int(e.tokens[0]) for e in entries]
        start = [e.request.length for e in entries]
        h[o[1]:o[2]] = start
        h[o[4]:o[5]] = start
        h[o[5]:o[6]] = [s + 1 for s in start]
        h[o[6]:o[7]] = [e.request.state_slot for e in entries]
        for gi in range(len(self.runner.cache.groups)):
            tab = h[o[8 + gi]:o[9 + gi]].reshape(B, W)
            for si, e in enumerate(entries):
                t = e.request.tables[gi]
                tab[si, :len(t)] = t
        self.dev.copy_(host, non_blocking=True)
        if self.copied[self.turn] is None:
            self.copied[self.turn] = torch.cuda.Event()
        self.copied[self.turn].record()
        self.runner.last_h2d_bytes = host.numel() * 4

    def run(self, entries: Sequence["StepEntry"]) -> torch.Tensor:
        from .. import kernels
        self.fill(entries)
        model = self.runner.model
        if self.graph is None:
            before = kernels.launches
            logits = model.forward(self.ctx, self.caches)          # this step, eagerly
            self.launches = kernels.launches - before
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            # No garbage collection while the stream is capturing: a collected object
            # that owns device memory, pinned memory or another graph would free it in
            # the middle of the capture and invalidate it.
            gc_was_on = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(graph):
                    self.logits = model.forward(self.ctx, self.caches)
            finally:
                if gc_was_on:
                    gc.enable()
            kernels.launches = before + self.launches              # recording launched nothing
            self.graph = graph
            return logits
        self.graph.replay()
        kernels.launches += self.launches
        return self.logits


class StepRunner:
    def __init__(self, model: DecoderModel, cache: CacheManager, max_step_tokens: int,
                 max_batch: int, max_seq: int, use_graphs: bool = True):
        self.model = model
        self.cache = cache
        self.max_step_tokens = int(max_step_tokens)
        self.max_batch = int(max_batch)
        self.max_seq = int(min(max_seq, model.spec.max_position))
        self.vocab = model.spec.vocab_size
        self.device = model.device
        self.steps = 0
        self.tokens_run = 0
        self.last_h2d_bytes = 0     # bytes of the last step's host-to-device copy
        self.use_graphs = bool(use_graphs) and self.device.type == "cuda" and getattr(model, "graph_safe", True)
        self.graphs = {}            # batch size -> GraphedDecode
        # what the sampler chose last for every request slot: a step may be launched
        # before the host has read the tokens of the step before
        self.last_token = torch.zeros(cache.max_requests, dtype=torch.int32, device=self.device)
        self.last_ctx = None        # the batch of the step that ran last, as the device holds it

    # ---- validation --------------------------------------------------------
    def release_graphs(self) -> None:
        """Drop the captured decode graphs and their static buffers now, not whenever
        the garbage collector finds them."""
        self.graphs.clear()

    def validate(self, entries: Sequence[StepEntry]) -> None:
        if not entries:
            raise StepError("a step needs at least one entry")
        if len(entries) > self.max_batch:
            raise StepError(f"{len(entries)} requests in one step, the batch limit is {self.max_batch}")
        seen = set()
        total = 0
        for e in entries:
            r = e.request
            if r.closed or self.cache.live.get(r.rid) is not r:
                raise StepError(f"request {r.rid} is not open")
            if r.rid in seen:
                raise StepError(f"request {r.rid} appears twice in one step")
            seen.add(r.rid)
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {r.rid} brings no tokens")
            if r.length + n > self.max_seq:
                raise StepError(f"request {r.rid}: positions [{r.length},{r.length + n}) exceed the "
                                f"sequence limit {self.max_seq}")
            if e.deferred and n != 1:
                raise StepError(f"request {r.rid}: a deferred entry brings exactly one token")
            for t in (() if e.deferred else e.tokens):
                if not (0 <= int(t) < self.vocab):
                    raise StepError(f"request {r.rid}: token id {t} outside the vocabulary of {self.vocab}")
            for w in e.want:
                if not (0 <= int(w) < n):
                    raise StepError(f"request {r.rid}: wanted place {w} outside its {n} tokens")
            total += n
        if total > self.max_step_tokens:
            raise StepError(f"{total} tokens in one step, the budget is {self.max_step_tokens}")

    # ---- the batch on the device ---------------------------------------------
    def build_context(self, entries: Sequence[StepEntry]) -> StepContext:
        S = len(entries)
        n_new = [len(e.tokens) for e in entries]
        start = [e.request.length for e in entries]
        n = sum(n_new)
        want_rows: List[int] = []
        q_start = [0]
        for e, cnt in zip(entries, n_new):
            want_rows.extend(q_start[-1] + int(w) for w in e.want)
            q_start.append(q_start[-1] + cnt)
        R = len(want_rows)
        widths = []
        for gi in range(len(self.cache.groups)):
            widths.append(max(1, max(len(e.request.tables[gi]) for e in entries)))
        sizes = [n, n, n, S + 1, S, S, S, max(R, 1)] + [S * w for w in widths]
        offs = np.concatenate([[0], np.cumsum(sizes)])
        host = torch.empty(int(offs[-1]), dtype=torch.int32, pin_memory=self.device.type == "cuda")
        h = host.numpy()
        h[offs[0]:offs[1]] = np.fromiter((-(e.request.state_slot + 1) if e.deferred else int(t)
                                          for e in entries for t in e.tokens), dtype=np.int32, count=n)
        h[offs[1]:offs[2]] = np.concatenate([np.arange(s, s + c, dtype=np.int32) for s, c in zip(start, n_new)])
        h[offs[2]:offs[3]] = np.repeat(np.arange(S, dtype=np.int32), n_new)
        h[offs[3]:offs[4]] = q_start
        h[offs[4]:offs[5]] = start
        h[offs[5]:offs[6]] = [s + c for s, c in zip(start, n_new)]
        h[offs[6]:offs[7]] = [e.request.state_slot for e in entries]
        h[offs[7]:offs[8]] = (want_rows + [0] * (max(R, 1) - R))
        for gi, w in enumerate(widths):
            tab = np.full((S, w), -1, dtype=np.int32)
            for si, e in enumerate(entries):
                t = e.request.tables[gi]
                tab[si, :len(t)] = t
            h[offs[8 + gi]:offs[9 + gi]] = tab.reshape(-1)
        dev = host.to(self.device, non_blocking=True)
        self.last_h2d_bytes = host.numel() * 4

        def part(i):
            return dev[int(offs[i]):int(offs[i + 1])]

        tables = {gi: part(8 + gi).view(S, w) for gi, w in enumerate(widths)}
        return StepContext(
            n_tokens=n, n_requests=S, token_ids=part(0), positions=part(1), token_req=part(2),
            q_start=part(3), start_pos=part(4), ctx_len=part(5), state_slots=part(6),
            block_tables=tables, want_rows=part(7)[:R], n_want=R,
            host_n_new=n_new, host_start_pos=start, max_new=max(n_new),
            max_ctx=max(s + c for s, c in zip(start, n_new)), all_single=all(c == 1 for c in n_new),
            last_token=self.last_token)

    # ---- run ---------------------------------------------------------------
    def run(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Logits float32 [wanted, vocab] on the device, in the order of the entries
        and of each entry's ``want``; None if nothing is wanted.  They stay valid until
        the next step (a replayed decode step reuses its buffer).  Raises ``StepError``
        for an invalid batch and ``OutOfPages`` when the cache cannot hold it; in both
        cases nothing has changed."""
        self.validate(entries)
        wants = [(e.request, len(e.tokens)) for e in entries]
        if not self.cache.can_reserve_all(wants):
            raise OutOfPages(f"the step's {sum(n for _, n in wants)} tokens do not fit the free pages "
                             f"{self.cache.free_pages()}")
        for r, n in wants:
            self.cache.reserve(r, n)
        try:
            if self.use_graphs and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries):
                g = self.graphs.get(len(entries))
                if g is None:
                    g = self.graphs[len(entries)] = GraphedDecode(self, len(entries))
                logits = g.run(entries)
                self.last_ctx = g.ctx
            else:
                ctx = self.build_context(entries)
                logits = self.model.forward(ctx, self.cache.layer_caches(ctx.block_tables))
                self.last_ctx = ctx
        except Exception:
            for r, _ in wants:
                self.cache.trim_reservation(r)
            raise
        for r, n in wants:
            self.cache.commit(r, n)
        self.steps += 1
        self.tokens_run += sum(n for _, n in wants)
        return logits
