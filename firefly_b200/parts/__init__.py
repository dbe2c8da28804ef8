from . import attention, block, embedding, mlp, norm, position  # noqa: F401  (registration)
from .base import CATEGORIES, Part, Runtime, build_part, part_class, register_part

__all__ = ["CATEGORIES", "Part", "Runtime", "build_part", "part_class", "register_part"]
