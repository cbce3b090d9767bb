from . import (attention, block, conv_attention, conv_filter, delta_rule, embedding, latent_attention, linear_attention, loop, mlp, moe, norm, parallel, position,
               state_space, token_side, wkv)  # noqa: F401  (registration)
from .base import CATEGORIES, Part, Runtime, build_part, part_class, register_part

__all__ = ["CATEGORIES", "Part", "Runtime", "build_part", "part_class", "register_part"]
