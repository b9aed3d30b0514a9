"""``DecoderModel``: a model assembled from a ``ModelSpec``.

It owns the parts (embedding, blocks, final norm, head), the list of tensors they
expect, and the forward pass of one step: embed the step's tokens, run the layer
calls of the schedule in order, each with its own view of the cache, add what is
pending and normalise the rows whose logits are wanted, and apply the head to
those rows only (the reference keeps each request's last row,
backend/model.cu:1181-1188; here the caller names the rows).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

# registering the built-in part kinds
from . import attention, block, embedding, mlp, norm, rotary  # noqa: F401
from .context import LayerCache, StepContext
from .spec import BuildEnv, ModelSpec, PagedKVNeed, StateNeed, TensorSpec, part_factory


class DecoderModel:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        env = BuildEnv(dtype=dtype, device=self.device, hidden_size=spec.hidden_size,
                       max_position=spec.max_position)
        self.env = env
        self.embedding = part_factory("embedding", spec.embedding.kind)(spec.embedding, env)
        self.blocks = [part_factory("block", b.kind)(b, env) for b in spec.blocks]
        self.final_norm = part_factory("norm", spec.final_norm.kind)(spec.final_norm, env)
        self.head = part_factory("head", spec.head.kind)(spec.head, env)
        self.schedule = list(spec.schedule)
        self._check_schedule()

    def _check_schedule(self):
        writers: Dict[int, int] = {}
        for i, call in enumerate(self.schedule):
            if not (0 <= call.block < len(self.blocks)):
                raise ValueError(f"schedule entry {i} names block {call.block} of {len(self.blocks)}")
            if call.writes_cache:
                if call.cache in writers:
                    raise ValueError(f"cache slot {call.cache} is written by schedule entries "
                                     f"{writers[call.cache]} and {i}")
                writers[call.cache] = i
        for i, call in enumerate(self.schedule):
            if not call.writes_cache and (call.cache not in writers or writers[call.cache] > i):
                raise ValueError(f"schedule entry {i} reads cache slot {call.cache} before a layer wrote it")
        slots = sorted(writers)
        if slots != list(range(len(slots))):
            raise ValueError(f"cache slots must be numbered 0..n-1, got {slots}")
        self.n_cache_slots = len(slots)
        self._writer_block = {slot: self.schedule[i].block for slot, i in writers.items()}

    # ---- weights ---------------------------------------------------------
    def parts(self):
        return [self.embedding] + self.blocks + [self.final_norm, self.head]

    def tensor_specs(self) -> List[TensorSpec]:
        seen: Dict[str, TensorSpec] = {}
        for p in self.parts():
            for s in p.tensor_specs():
                if s.name in seen and seen[s.name].shape != s.shape:
                    raise ValueError(f"tensor {s.name} is declared with two shapes")
                seen.setdefault(s.name, s)
        return list(seen.values())

    @property
    def graph_safe(self) -> bool:
        """False when a part says that its forward cannot be captured into a CUDA graph
        (class or instance attribute ``graph_safe = False``: it reads device data on the
        host, or its shapes depend on the data)."""
        return all(getattr(p, "graph_safe", True) for p in self.parts())

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self.parts():
            p.bind(tensors)
        # a block may warm the cache for the block that the schedule runs after it
        # (first successor wins where a block runs more than once)
        told = set()
        for call, nxt in zip(self.schedule, self.schedule[1:]):
            tell = getattr(self.blocks[call.block], "set_successor", None)
            if tell is not None and call.block not in told:
                told.add(call.block)
                tell(self.blocks[nxt.block])

    # ---- cache -----------------------------------------------------------
    def cache_needs(self):
        """For every cache slot, what the mixer that writes it asks for."""
        needs = []
        for slot in range(self.n_cache_slots):
            mixer = self.blocks[self._writer_block[slot]].mixer
            needs.append(mixer.cache_need())
        return needs

    # ---- one step --------------------------------------------------------
    def forward(self, ctx: StepContext, caches: List[LayerCache]) -> Optional[torch.Tensor]:
        """Logits float32 [ctx.n_want, vocab] at ``ctx.want_rows`` (None when no row
        is wanted; the cache is still filled)."""
        x = self.embedding.forward(ctx.token_ids, ctx.last_token)
        pending = None
        for call in self.schedule:
            cache = caches[call.cache]
            if cache.writes != call.writes_cache:
                cache = LayerCache(cache.k, cache.v, cache.block_table, cache.state,
                                   writes=call.writes_cache, page_size=cache.page_size)
            pending = self.blocks[call.block].forward(x, pending, ctx, cache)
        if ctx.n_want == 0:
            return None
        if pending is None and hasattr(self.head, "forward_normed"):
            logits = self.head.forward_normed(x, self.final_norm, ctx.want_rows)
            if logits is not None:
                return logits
        xn = self.final_norm.forward(x, pending, rows=ctx.want_rows)
        return self.head.forward(xn)
