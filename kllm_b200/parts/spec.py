"""Descriptions from which a model is assembled, and the registries of part kinds.

An architecture turns its typed configuration into a ``ModelSpec``: plain data that
names, layer by layer, which mixer, feed-forward, norm and block arrangement to
build, with every size and constant as a parameter, and in which order the layers
run.  ``kllm_b200.parts.model.DecoderModel`` builds the parts through the
registries below; no part is told which model it is in.

The order of execution is data too: ``ModelSpec.schedule`` is a list of
``LayerCall(block, cache, writes_cache)``.  A block index may appear twice (the
same weights run again, each call with a cache slot of its own), and a call may
name the cache slot of another call with ``writes_cache=False`` to read keys and
values that an earlier layer wrote.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class TensorSpec:
    """One tensor a part expects from the weight files.

    store: "compute" -> kept in the model's dtype (bfloat16 or float32);
           "float32" -> kept in 32-bit whatever the model's dtype (norm gains,
           router tables); "int32" -> integer table.
    init:  how random-weights mode fills it: "normal" (mean 0), "gain" (mean 1) or
           "zeros"; the spreads are arguments of that mode.
    optional: may be absent from the files (the part then copes, e.g. a tied head).
    """
    name: str
    shape: Tuple[int, ...]
    store: str = "compute"
    init: str = "normal"
    optional: bool = False


@dataclass
class PartSpec:
    kind: str
    prefix: str = ""
    params: Dict = field(default_factory=dict)


@dataclass
class BlockSpec:
    """One layer: an arrangement (``kind``) of a mixer, a feed-forward and norms."""
    kind: str
    prefix: str
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    ff_norm: PartSpec
    params: Dict = field(default_factory=dict)


@dataclass(frozen=True)
class LayerCall:
    block: int
    cache: int
    writes_cache: bool = True


@dataclass
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_position: int
    embedding: PartSpec
    blocks: List[BlockSpec]
    schedule: List[LayerCall]
    final_norm: PartSpec
    head: PartSpec
    eos_token_ids: Tuple[int, ...] = ()


# ---- what a mixer asks of the cache manager ---------------------------------

@dataclass(frozen=True)
class PagedKVNeed:
    """Keys and values in pages.  window None: every key is kept; window W: only
    the last W keys of a request are ever read, older pages may be given back."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size, one slot per live request, zero at the
    start of a request."""
    shape: Tuple[int, ...]
    dtype: str = "float32"


# ---- registries -----------------------------------------------------------

_KINDS: Dict[str, Dict[str, Callable]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "qk_transform": {}, "block": {},
    "embedding": {}, "head": {},
}


def register_part(family: str, kind: str, factory: Callable) -> None:
    """``factory(spec: PartSpec, env: BuildEnv)`` returns the part.  ``family`` is one
    of mixer, feed_forward, norm, position, qk_transform, block, embedding, head."""
    if family not in _KINDS:
        raise KeyError(f"unknown part family {family!r}; families: {sorted(_KINDS)}")
    _KINDS[family][kind] = factory


def part_factory(family: str, kind: str) -> Callable:
    try:
        return _KINDS[family][kind]
    except KeyError:
        raise KeyError(f"no {family} of kind {kind!r} is registered; known: "
                       f"{sorted(_KINDS.get(family, {}))}") from None


@dataclass
class BuildEnv:
    """What every part is given at construction."""
    dtype: "object"      # torch.dtype of weights, activations and cache
    device: "object"     # torch.device
    hidden_size: int
    max_position: int
