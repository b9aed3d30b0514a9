"""Gated feed-forward (SwiGLU): down( act(x Wg^T) * (x Wu^T) ).

params: ``hidden``, ``intermediate``, ``activation`` ("silu").  Tensors:
``<prefix>.{gate,up}_proj.weight`` [f, d] and ``<prefix>.down_proj.weight`` [d, f],
no bias (reference backend/model.cu:1112-1115, activation :477-483).  Gate and up
are stacked into one [2f, d] matrix at bind time so both are one product.

Optional ``forward_residual(x, norm, ctx) -> bool``: as for mixers, the part reads
the float32 residual stream, applies ``norm`` inside its first kernel and adds its
result into x, or returns False.  Here, for steps of a few tokens, the gate/up
product carries the norm as prologue and the activation as epilogue, the down
product adds into x (csrc/skinny_gemm.cu).  Large portions in bfloat16 run gate, up
and the activation as one tensor-core kernel (csrc/gemm_tcgen05.cu) where its tiles
fill the GPU; everything else uses the library product and the activation kernel.

Interface of a feed-forward part: ``forward(xn, ctx) -> [n, hidden]`` in float32 or
the model dtype.
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
        self._after = []           # weights streamed right after this part (see set_prefetch_targets)

    def tensor_specs(self):
        return [TensorSpec(f"{self.prefix}.gate_proj.weight", (self.inter, self.hidden)),
                TensorSpec(f"{self.prefix}.up_proj.weight", (self.inter, self.hidden)),
                TensorSpec(f"{self.prefix}.down_proj.weight", (self.hidden, self.inter))]

    def bind(self, tensors):
        self.w_gate_up = torch.cat([tensors[f"{self.prefix}.gate_proj.weight"],
                                    tensors[f"{self.prefix}.up_proj.weight"]], dim=0).contiguous()
        self.w_down = tensors[f"{self.prefix}.down_proj.weight"]

    def streamed_weights(self):
        """The matrices this part streams in a small step, in kernel order."""
        return [self.w_gate_up, self.w_down]

    def set_prefetch_targets(self, weights):
        """What the kernels after this part stream first (the next layer's mixer's
        ``streamed_weights``): in a small step this part's two kernels ask for them
        to be brought into L2 while they run."""
        self._after = list(weights)

    def _target(self, i):
        return self._after[i] if i < len(self._after) else None

    def _activation(self, xn):
        """silu(gate) * up as a matrix of the model dtype."""
        n = xn.shape[0]
        act = torch.empty((n, self.inter), dtype=self.dtype, device=xn.device)
        w_gate, w_up = self.w_gate_up[:self.inter], self.w_gate_up[self.inter:]
        if (self.dtype == torch.bfloat16 and kernels.gemm_pays(n, self.inter, "swiglu")
                and kernels.gemm_fits(xn, w_gate, act, "swiglu", w_up)):
            # large portions: both products and the activation in one tcgen05 kernel
            kernels.gemm(xn, w_gate, weight_up=w_up, epilogue="swiglu", out=act)
        else:
            gu = kernels.linear(xn, self.w_gate_up, out_dtype=torch.float32)
            kernels.silu_mul(act, gu[:, :self.inter], gu[:, self.inter:])
        return act

    def forward(self, xn, ctx):
        # gate and up stay float32 until the activation has been applied; the down
        # projection's float32 result goes into the residual stream unrounded
        act = self._activation(xn)
        return kernels.linear(act, self.w_down, out_dtype=torch.float32)


    def forward_residual(self, x, norm, ctx):
        n = x.shape[0]
        if not (getattr(norm, "fusable_rmsnorm", False) and kernels.skinny_fits(n, self.hidden, self.dtype)
                and kernels.skinny_fits(n, self.inter, self.dtype, sliced=True)):
            # larger steps: the down product adds into the residual stream
            kernels.linear_add(x, self._activation(norm.forward(x, None)), self.w_down)
            return True
        act = kernels.skinny_gemm(self.w_gate_up[:self.inter], weight_up=self.w_gate_up[self.inter:], x_f32=x,
                                  gain=norm.gain, eps=norm.eps, epilogue="swiglu", prefetch=self._target(0))
        kernels.skinny_gemm(self.w_down, x=act, epilogue="add", out=x, prefetch=self._target(1))
        return True


register_part("feed_forward", "gated_mlp", GatedMLP)
