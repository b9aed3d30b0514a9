"""Token embedding and output head.

Embedding: params ``vocab``, ``width``; tensor ``<prefix>.weight`` [vocab, width];
``forward(ids) -> x`` float32 [n, width], the residual stream (reference
backend/model.cu:89-95, no scaling for Llama).

Head: params ``vocab``, ``width``, ``tied_to`` (name of the embedding tensor to
share, or None); tensor ``<prefix>.weight`` [vocab, width] unless tied;
``forward(xn) -> logits`` float32 [rows, vocab], accumulated in float32 (reference
backend/model.cu:1187; tying resolved offline there, tools/convert_hf.py:81-82).
"""
from __future__ import annotations

import torch

from .. import kernels
from .spec import BuildEnv, PartSpec, TensorSpec, register_part


class TokenEmbedding:
    def __init__(self, spec: PartSpec, env: BuildEnv):
        self.vocab = int(spec.params["vocab"])
        self.width = int(spec.params["width"])
        self.name = spec.prefix + ".weight"
        self.table = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.vocab, self.width))]

    def bind(self, tensors):
        self.table = tensors[self.name]

    def forward(self, ids, last_token=None):
        x = torch.empty((ids.numel(), self.width), dtype=torch.float32, device=ids.device)
        kernels.embed(x, self.table, ids, last_token)
        return x


class LinearHead:
    def __init__(self, spec: PartSpec, env: BuildEnv):
        self.vocab = int(spec.params["vocab"])
        self.width = int(spec.params["width"])
        self.tied_to = spec.params.get("tied_to")
        self.name = spec.prefix + ".weight"
        self.weight = None

    def tensor_specs(self):
        # a tied model's files may still carry a copy of the head; it is not used
        return [TensorSpec(self.name, (self.vocab, self.width), optional=bool(self.tied_to))]

    def bind(self, tensors):
        self.weight = tensors[self.tied_to] if self.tied_to else tensors[self.name]

    def forward(self, xn):
        return kernels.linear(xn, self.weight, out_dtype=torch.float32)

    def forward_normed(self, x, norm, rows):
        """Logits of rows ``rows`` of the float32 residual stream with ``norm`` applied
        inside the product, or None when that route does not fit."""
        n = rows.numel()
        if not (getattr(norm, "fusable_rmsnorm", False) and kernels.skinny_fits(n, self.width, self.weight.dtype)):
            return None
        return kernels.skinny_gemm(self.weight, x_f32=x, gain=norm.gain, eps=norm.eps, rows=rows, epilogue="f32")


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "linear_head", LinearHead)
