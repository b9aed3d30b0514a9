"""Gated feed-forward (SwiGLU): down( act(x Wg^T) * (x Wu^T) ).

params: ``hidden``, ``intermediate``, ``activation`` ("silu").  Tensors:
``<prefix>.{gate,up}_proj.weight`` [f, d] and ``<prefix>.down_proj.weight`` [d, f],
no bias (reference backend/model.cu:1112-1115, activation :477-483).  Gate and up
are stacked into one [2f, d] matrix at bind time so both are one product.

Interface of a feed-forward part: ``forward(xn, ctx) -> [n, hidden]`` in the model
dtype.
"""
from __future__ import annotations

import torch

from .. import kernels
from .spec import BuildEnv, PartSpec, TensorSpec, register_part


class GatedMLP:
    def __init__(self, spec: PartSpec, env: BuildEnv):
        p = spec.params
        self.hidden = int(p["hidden"])
        self.inter = int(p["intermediate"])
        self.activation = p.get("activation", "silu")
        if self.activation != "silu":
            raise ValueError(f"gated feed-forward: activation {self.activation!r} has no kernel (silu only)")
        self.prefix = spec.prefix
        self.dtype = env.dtype
        self.w_gate_up = None
        self.w_down = None

    def tensor_specs(self):
        return [TensorSpec(f"{self.prefix}.gate_proj.weight", (self.inter, self.hidden)),
                TensorSpec(f"{self.prefix}.up_proj.weight", (self.inter, self.hidden)),
                TensorSpec(f"{self.prefix}.down_proj.weight", (self.hidden, self.inter))]

    def bind(self, tensors):
        self.w_gate_up = torch.cat([tensors[f"{self.prefix}.gate_proj.weight"],
                                    tensors[f"{self.prefix}.up_proj.weight"]], dim=0).contiguous()
        self.w_down = tensors[f"{self.prefix}.down_proj.weight"]

    def forward(self, xn, ctx):
        gu = kernels.linear(xn, self.w_gate_up)
        act = torch.empty((xn.shape[0], self.inter), dtype=self.dtype, device=xn.device)
        kernels.silu_mul(act, gu[:, :self.inter], gu[:, self.inter:])
        return kernels.linear(act, self.w_down)


register_part("feed_forward", "gated_mlp", GatedMLP)
