from .base import (CATEGORIES, Runtime, build_part, part_class, part_tensors, register_part)
from . import (norm, position, attention, talking_attention, latent_attention, linear_attention, side_by_side, conv, ssm,
               delta_rule, mlp,
               token_input, block, embed_head)  # noqa: F401  (registration)
from .linear import Linear

__all__ = ["CATEGORIES", "Runtime", "build_part", "part_class", "part_tensors", "register_part",
           "Linear"]
