from . import attention, block, embedding, feed_forward, norm, position  # noqa: F401 (register kinds)
from .base import (CacheNeed, ParamInfo, Part, ResidualStream, StateNeed, build_part, part_class,
                   register_part)

__all__ = ["CacheNeed", "ParamInfo", "Part", "ResidualStream", "StateNeed", "build_part", "part_class",
           "register_part"]
