from .base import (Block, BuildContext, CacheNeeds, FeedForward, LogitsPost, Mixer, Norm, PagedKVNeed, Part,
                   PositionEncoding, SlotStateNeed, Workspace)
from .registry import build, build_block, build_norm, kinds, register, unregister

__all__ = [
    "Block", "BuildContext", "CacheNeeds", "FeedForward", "LogitsPost", "Mixer", "Norm", "PagedKVNeed", "Part",
    "PositionEncoding", "SlotStateNeed", "Workspace", "build", "build_block", "build_norm",
    "kinds", "register", "unregister",
]
