"""Causal grouped-query attention over a paged cache: the mixer of a Llama layer.

params: ``hidden``, ``n_heads``, ``n_kv_heads``, ``head_dim``; optional ``window``
(None: every earlier key is visible; W: the last W keys, the query's own included),
``scale`` (default 1/sqrt(head_dim)), ``position`` (a PartSpec of the position
family, e.g. rotary; None for no position encoding), ``qk_transform`` (a PartSpec of
the qk_transform family, None for Llama: something applied to the projected queries
and keys before the position encoding, such as a norm per head or a bias; interface
``tensor_specs()``, ``bind(tensors)``, ``apply(q, k, ctx, n_heads, n_kv_heads,
head_dim)`` which changes q [n, H*hd] and k [n, G*hd] (None when the layer reads
another layer's cache) in place; with one, a decode step takes the separate rotary
and attention kernels, since the fused kernel rotates the raw projections itself),
``score_slopes`` (a list of one float per head, None for Llama: slope[h] * (key
position - query position) is added to the scaled scores, the form of position
encodings that act on the scores; such a layer runs the CUDA-core attention kernel, the
only one that takes the argument).
Tensors: ``<prefix>.{q,k,v,o}_proj.weight`` with shapes [H*hd, d], [G*hd, d],
[G*hd, d], [d, H*hd]; no bias (reference backend/model.cu:1090-1104).  At bind time
q, k and v are stacked into one [(H+2G)*hd, d] matrix so the three projections are
one product.

Interface of a mixer part:
  ``cache_need()`` -> PagedKVNeed | StateNeed | None
  ``forward(xn, ctx, cache) -> [n, hidden]`` in float32 or the model dtype, xn being
  the normed input [n, hidden]; the residual sum is the block's business.
  Optional: ``forward_residual(x, norm, ctx, cache) -> bool`` takes the float32
  residual stream itself, applies ``norm`` inside its first kernel and adds its
  result into x; it returns False when it cannot (sizes, dtype, kind of norm) and
  the block then takes the general route.  Here it serves steps of a few tokens
  (decode): both projections become weight-streaming products with the norm as
  prologue and the residual sum as epilogue (csrc/skinny_gemm.cu).
The new keys and values of a step are written to the pages before attention runs,
so a query sees the keys of its own portion through the cache, like every other
key (reference :1096-1102).
"""
from __future__ import annotations

import math

import torch

from .. import kernels
from .spec import BuildEnv, PagedKVNeed, PartSpec, TensorSpec, part_factory, register_part


class PagedAttention:
    def __init__(self, spec: PartSpec, env: BuildEnv):
        p = spec.params
        self.hidden = int(p["hidden"])
        self.n_heads = int(p["n_heads"])
        self.n_kv = int(p["n_kv_heads"])
        self.head_dim = int(p["head_dim"])
        if self.n_heads % self.n_kv:
            raise ValueError(f"{self.n_heads} heads are not a multiple of {self.n_kv} kv heads")
        self.window = p.get("window")
        self.scale = float(p.get("scale") or 1.0 / math.sqrt(self.head_dim))
        self.q_dim = self.n_heads * self.head_dim
        self.kv_dim = self.n_kv * self.head_dim
        self.prefix = spec.prefix
        self.dtype = env.dtype
        pos = p.get("position")
        self.position = part_factory("position", pos.kind)(pos, env) if pos is not None else None
        qt = p.get("qk_transform")
        self.qk_transform = part_factory("qk_transform", qt.kind)(qt, env) if qt is not None else None
        slopes = p.get("score_slopes")
        if slopes is not None and len(slopes) != self.n_heads:
            raise ValueError(f"score_slopes: {len(slopes)} values for {self.n_heads} heads")
        self.score_slopes = None if slopes is None else torch.tensor([float(v) for v in slopes], dtype=torch.float32,
                                                                     device=env.device)
        self.w_qkv = None
        self.w_o = None
        # Zeroed scratch of the fused decode kernel, which leaves it zero.  A captured decode
        # graph holds the address of the buffer it was recorded with, so a buffer is never
        # freed once it has been used: a larger step gets a new one and the old ones stay.
        self._counters = None
        self._counters_kept = []
        self._after = []           # weights streamed right after this part (see set_prefetch_targets)

    def _names(self):
        return {k: f"{self.prefix}.{k}_proj.weight" for k in "qkvo"}

    def tensor_specs(self):
        n = self._names()
        return [TensorSpec(n["q"], (self.q_dim, self.hidden)),
                TensorSpec(n["k"], (self.kv_dim, self.hidden)),
                TensorSpec(n["v"], (self.kv_dim, self.hidden)),
                TensorSpec(n["o"], (self.hidden, self.q_dim))] + \
            (self.position.tensor_specs() if self.position else []) + \
            (self.qk_transform.tensor_specs() if self.qk_transform else [])

    def bind(self, tensors):
        n = self._names()
        self.w_qkv = torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]], dim=0).contiguous()
        self.w_o = tensors[n["o"]]
        if self.position:
            self.position.bind(tensors)
        if self.qk_transform:
            self.qk_transform.bind(tensors)

    def cache_need(self):
        return PagedKVNeed(self.n_kv, self.head_dim, self.window)

    def _split(self, qkv, writes):
        q = qkv[:, :self.q_dim]
        if not writes:
            return q, q, q
        return q, qkv[:, self.q_dim:self.q_dim + self.kv_dim], qkv[:, self.q_dim + self.kv_dim:]

    def streamed_weights(self):
        """The matrices this part streams in a small step, in kernel order."""
        return [self.w_qkv, self.w_o]

    def set_prefetch_targets(self, weights):
        """What the kernels after this part stream first (the next part's
        ``streamed_weights``): in a small step the attention kernel and the output
        projection ask for them to be brought into L2 while they run."""
        self._after = list(weights)

    def _target(self, i):
        return self._after[i] if i < len(self._after) else None

    def _attend(self, q, k, v, ctx, cache, prefetch=None):
        n = q.shape[0]
        group = self.n_heads // self.n_kv
        table = getattr(self.position, "full_rotary_table", lambda: None)() if self.position is not None else None
        if self.qk_transform is not None:
            self.qk_transform.apply(q, k if cache.writes else None, ctx, self.n_heads, self.n_kv, self.head_dim)
            table = None          # the fused decode kernel takes the raw projections
        if self.score_slopes is not None:
            table = None          # ... and has no bias on its scores
        if (table is not None and cache.writes and ctx.all_single and self.dtype == torch.bfloat16 and group <= 16
                and self.head_dim in kernels.TC_HEAD_DIMS and self.head_dim % 32 == 0):
            # decode: rotary encoding, cache write and attention in one kernel
            if self._counters is None or self._counters.numel() < n * self.n_kv:
                if self._counters is not None:
                    self._counters_kept.append(self._counters)
                self._counters = torch.zeros(max(256, 2 * n) * self.n_kv, dtype=torch.int32, device=q.device)
            attn = torch.empty((n, self.q_dim), dtype=self.dtype, device=q.device)
            kernels.attention_decode_fused(
                attn, q, k, v, table, cache.k, cache.v, ctx.positions, None, cache.block_table,   # token t is request t
                self._counters, self.n_heads, self.n_kv, self.head_dim, self.window or 0, self.scale,
                kernels.decode_splits(n, self.n_kv, ctx.split_bound or ctx.max_ctx), prefetch=prefetch)
            return attn
        if self.position is not None:
            self.position.apply(q, k, v, ctx, cache, self.n_heads, self.n_kv)
        elif cache.writes:
            kernels.rope_append(q, k, v, None, ctx.positions, ctx.token_req, cache.block_table,
                                cache.k, cache.v, self.n_heads, self.n_kv, self.head_dim)
        attn = torch.empty((n, self.q_dim), dtype=self.dtype, device=q.device)
        kernels.attention(attn, q, cache.k, cache.v, ctx, cache.block_table, self.n_heads, self.n_kv,
                          self.head_dim, self.window or 0, self.scale, score_slopes=self.score_slopes)
        return attn

    def forward(self, xn, ctx, cache):
        # a layer that reads another layer's cache projects its queries only
        w = self.w_qkv if cache.writes else self.w_qkv[:self.q_dim]
        q, k, v = self._split(kernels.linear(xn, w), cache.writes)
        attn = self._attend(q, k, v, ctx, cache)
        # float32 out: the result goes into the residual stream unrounded
        return kernels.linear(attn, self.w_o, out_dtype=torch.float32)

    def forward_residual(self, x, norm, ctx, cache):
        n = x.shape[0]
        w = self.w_qkv if cache.writes else self.w_qkv[:self.q_dim]
        if not (getattr(norm, "fusable_rmsnorm", False) and kernels.skinny_fits(n, self.hidden, self.dtype)
                and kernels.skinny_fits(n, self.q_dim, self.dtype, sliced=True)):
            # larger steps: the library's products, the last one adding into the residual stream
            q, k, v = self._split(kernels.linear(norm.forward(x, None), w), cache.writes)
            kernels.linear_add(x, self._attend(q, k, v, ctx, cache), self.w_o)
            return True
        qkv = kernels.skinny_gemm(w, x_f32=x, gain=norm.gain, eps=norm.eps, epilogue="store")
        q, k, v = self._split(qkv, cache.writes)
        attn = self._attend(q, k, v, ctx, cache, prefetch=self._target(0))
        kernels.skinny_gemm(self.w_o, x=attn, epilogue="add", out=x, prefetch=self._target(1))
        return True


register_part("mixer", "paged_attention", PagedAttention)
