from .base import (KVNeed, LayerIO, NormedInput, ParamDecl, Part, StateNeed, block_class, feed_forward_class, hook_class,
                   mixer_class, norm_class, position_class, register_block, register_feed_forward, register_hook,
                   register_mixer, register_norm, register_position, unregister)
from .linear import Linear
from . import norm, rope, attention, mlp, block  # noqa: F401  (registers the parts)

__all__ = [
    "KVNeed", "LayerIO", "ParamDecl", "Part", "StateNeed", "Linear",
    "block_class", "feed_forward_class", "hook_class", "mixer_class", "norm_class", "position_class",
    "register_block", "register_feed_forward", "register_hook", "register_mixer", "register_norm",
    "register_position",
    "unregister",
]
