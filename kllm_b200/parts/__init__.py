from .context import LayerCache, StepContext
from .spec import (BlockSpec, BuildEnv, LayerCall, ModelSpec, PagedKVNeed, PartSpec, StateNeed,
                   TensorSpec, part_factory, register_part)

__all__ = ["LayerCache", "StepContext", "BlockSpec", "BuildEnv", "LayerCall", "ModelSpec",
           "PagedKVNeed", "PartSpec", "StateNeed", "TensorSpec", "part_factory", "register_part"]

# the built-in part kinds register themselves on import
from . import attention, block, embedding, mlp, norm, rotary  # noqa: E402,F401
