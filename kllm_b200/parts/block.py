"""Arrangements of a layer's parts.

``pre_norm``: x += mixer(norm1(x)); x += ff(norm2(x)), with the feed-forward's
output handed on as ``pending`` and added inside the next norm (the next layer's
first norm, or the model's final norm), as the reference does
(backend/model.cu:1068-1072, 1083-1089, 1105, 1117).

Interface of a block: ``forward(x, pending, ctx, cache) -> pending'``.  x is the
float32 residual stream, updated in place; ``pending`` (float32 or model dtype, or
None) is what is still to be added to x.

A mixer or feed-forward may offer ``forward_residual`` (the part applies the norm and
adds its result into x itself, in whichever kernels fit the step's size); the block
uses it whenever nothing is pending.  The built-in attention and gated feed-forward
both offer it and always accept, so a Llama layer never hands anything on as
``pending``.  A part without it, or one that returns False, gets norm -> ``forward``
-> pending.  Both routes compute the same sums.

Two more optional methods let a part's kernels warm L2 for the kernels after them:
``streamed_weights()`` (the matrices a part streams in a small step, in kernel order)
and ``set_prefetch_targets(weights)`` (what runs right after the part).  The block
wires mixer -> feed-forward when it is bound, the model wires feed-forward -> the next
block's mixer through ``set_successor``.  A part without them is left alone.
"""
from __future__ import annotations

from .spec import BlockSpec, BuildEnv, part_factory, register_part


class PreNormBlock:
    def __init__(self, spec: BlockSpec, env: BuildEnv):
        self.mixer = part_factory("mixer", spec.mixer.kind)(spec.mixer, env)
        self.feed_forward = part_factory("feed_forward", spec.feed_forward.kind)(spec.feed_forward, env)
        self.mixer_norm = part_factory("norm", spec.mixer_norm.kind)(spec.mixer_norm, env)
        self.ff_norm = part_factory("norm", spec.ff_norm.kind)(spec.ff_norm, env)

    def parts(self):
        return [self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward]

    def tensor_specs(self):
        return [s for p in self.parts() for s in p.tensor_specs()]

    @property
    def graph_safe(self):
        return all(getattr(p, "graph_safe", True) for p in self.parts())

    def bind(self, tensors):
        for p in self.parts():
            p.bind(tensors)
        self._wire(self.mixer, self.feed_forward)

    @staticmethod
    def _wire(part, following):
        """Tell ``part`` which weights the part after it streams, if both take part in
        that (optional methods ``set_prefetch_targets`` / ``streamed_weights``)."""
        tell, ask = getattr(part, "set_prefetch_targets", None), getattr(following, "streamed_weights", None)
        if tell is not None and ask is not None:
            tell(ask())

    def set_successor(self, block):
        """The block that runs after this one in the model's schedule."""
        self._wire(self.feed_forward, getattr(block, "mixer", None))

    def forward(self, x, pending, ctx, cache):
        fused = getattr(self.mixer, "forward_residual", None)
        if pending is None and fused is not None and fused(x, self.mixer_norm, ctx, cache):
            pending = None
        else:
            xn = self.mixer_norm.forward(x, pending)
            pending = self.mixer.forward(xn, ctx, cache)
        fused = getattr(self.feed_forward, "forward_residual", None)
        if pending is None and fused is not None and fused(x, self.ff_norm, ctx):
            return None
        xn = self.ff_norm.forward(x, pending)
        return self.feed_forward.forward(xn, ctx)


register_part("block", "pre_norm", PreNormBlock)
