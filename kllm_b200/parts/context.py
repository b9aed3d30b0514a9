"""What a step hands to the parts: the batch laid out on the device, and the view
of the cache that one layer call works on."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch


@dataclass
class StepContext:
    """One batch of new tokens, all requests concatenated.

    Row t of every per-token tensor belongs to request ``token_req[t]`` (an index
    into this step's requests, not a global id) and sits at absolute position
    ``positions[t]`` of that request.  ``q_start[s] .. q_start[s+1]`` are the rows of
    request s; ``start_pos[s]`` is its cache length before the step and
    ``ctx_len[s]`` after it.  ``block_tables[g]`` is the [requests, max_blocks]
    table of cache group g (-1 where a request holds no page); ``state_slots[s]``
    is the request's slot in every per-request state tensor.  A negative token id
    -(slot + 1) stands for the token that was sampled for that request slot in the step
    before and is still on the device, in ``last_token[slot]``.
    """
    n_tokens: int
    n_requests: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    token_req: torch.Tensor
    q_start: torch.Tensor
    start_pos: torch.Tensor
    ctx_len: torch.Tensor
    state_slots: torch.Tensor
    block_tables: Dict[int, torch.Tensor]
    want_rows: torch.Tensor
    n_want: int
    # host-side copies for planning launches (never read by kernels)
    host_n_new: List[int] = field(default_factory=list)
    host_start_pos: List[int] = field(default_factory=list)
    max_new: int = 0
    max_ctx: int = 0
    all_single: bool = False   # every request brings exactly one token
    split_bound: int = 0       # context bound that fixes launch shapes (0: use max_ctx)
    last_token: Optional[torch.Tensor] = None   # int32 [request slots]: the sampler's latest choice per slot


@dataclass
class LayerCache:
    """The cache as one layer call sees it."""
    k: Optional[torch.Tensor]            # [pages, kv heads, page_size, head_dim]
    v: Optional[torch.Tensor]
    block_table: Optional[torch.Tensor]  # [requests, max_blocks] int32
    state: Optional[torch.Tensor]        # [slots, *state shape]
    writes: bool = True
    page_size: int = 0
