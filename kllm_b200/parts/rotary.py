"""Rotary position encoding (rotate_half convention).

params: ``head_dim``, ``theta``, optional ``rotary_dim`` (defaults to head_dim; a
smaller even value rotates only the first dims of each head).  The part owns a
float32 table [max_position, rotary_dim] of cos (first half of a row) and sin
(second half), computed in float64 from angle = p * theta^(-2j/rotary_dim), which is
how the reference forms its angles (backend/model.cu:176-178).

Interface of a position part used by the attention mixer:
``apply(q, k, v, ctx, cache, n_heads, n_kv_heads)`` rotates q in place and, when the
layer writes its cache, stores rotated k and v into the pages.  Optional:
``full_rotary_table()`` returns the cos/sin table when the whole head is rotated, for
a mixer whose kernel can do the rotation itself.
"""
from __future__ import annotations

import torch

from .. import kernels
from .spec import BuildEnv, PartSpec, register_part


class RotaryEmbedding:
    def __init__(self, spec: PartSpec, env: BuildEnv):
        self.head_dim = int(spec.params["head_dim"])
        self.theta = float(spec.params["theta"])
        self.rotary_dim = int(spec.params.get("rotary_dim", self.head_dim))
        if self.rotary_dim % 2 or not (0 < self.rotary_dim <= self.head_dim):
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and within head_dim {self.head_dim}")
        half = self.rotary_dim // 2
        j = torch.arange(half, dtype=torch.float64)
        freq = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * j / self.rotary_dim)
        ang = torch.arange(env.max_position, dtype=torch.float64)[:, None] * freq[None, :]
        table = torch.cat([torch.cos(ang), torch.sin(ang)], dim=1).to(torch.float32)
        self.cos_sin = table.contiguous().to(env.device)

    def tensor_specs(self):
        return []

    def bind(self, tensors):
        pass

    def full_rotary_table(self):
        return self.cos_sin if self.rotary_dim == self.head_dim else None

    def apply(self, q, k, v, ctx, cache, n_heads, n_kv_heads):
        writes = cache.writes and cache.k is not None
        kernels.rope_append(q, k, v, self.cos_sin, ctx.positions, ctx.token_req,
                            cache.block_table if writes else None,
                            cache.k if writes else None, cache.v if writes else None,
                            n_heads, n_kv_heads, self.head_dim)


register_part("position", "rotary", RotaryEmbedding)
