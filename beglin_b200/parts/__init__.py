"""The parts a model is put together from, and their registries.  Importing this package registers
the built-in parts."""
from . import attention, block, mlp, norm, rope  # noqa: F401  (registration)
from .cache_need import FixedStateNeed, FixedStateView, PagedKVNeed, PagedKVView
from .context import BuildContext
from .linear import Linear
from .registry import (register_block, register_feed_forward, register_mixer, register_norm,
                       register_position)
from .spec import (AttentionSpec, LayerSpec, ModelSpec, NormSpec, PositionSpec, Stage, SwiGLUSpec,
                   TensorRole)

__all__ = ["FixedStateNeed", "FixedStateView", "PagedKVNeed", "PagedKVView", "BuildContext", "Linear",
           "register_block", "register_feed_forward", "register_mixer", "register_norm",
           "register_position", "AttentionSpec", "LayerSpec", "ModelSpec", "NormSpec", "PositionSpec",
           "Stage", "SwiGLUSpec", "TensorRole"]
