"""RMSNorm with the residual sum folded in.

params: ``width``, ``eps``.  Tensor: ``<prefix>.weight`` [width], kept in float32
(reference backend/model.cu:101-122, 144-165; the gain is used as stored, no 1 + w).
Interface of a norm part:
``forward(x, res, rows=None) -> out``: x is the float32 residual stream [n, width];
``res`` (float32 or model dtype, or None) is added into x first and x is written back; the
result is in the model dtype.  With ``rows`` only those rows are normalised and x
is left as it is.

A part that can apply this norm inside its own kernel (see ``forward_residual`` of
the attention and feed-forward parts) recognises it by ``fusable_rmsnorm`` and
reads ``gain`` and ``eps``.
"""
from __future__ import annotations

import torch

from .. import kernels
from .spec import BuildEnv, PartSpec, TensorSpec, register_part


class RMSNorm:
    fusable_rmsnorm = True

    def __init__(self, spec: PartSpec, env: BuildEnv):
        self.width = int(spec.params["width"])
        self.eps = float(spec.params["eps"])
        self.name = spec.prefix + ".weight"
        self.dtype = env.dtype
        self.gain = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.width,), store="float32", init="gain")]

    def bind(self, tensors):
        self.gain = tensors[self.name]

    def forward(self, x, res=None, rows=None):
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.width), dtype=self.dtype, device=x.device)
        kernels.add_rmsnorm(x, res, out, self.gain, self.eps, rows=rows)
        return out


register_part("norm", "rmsnorm", RMSNorm)
