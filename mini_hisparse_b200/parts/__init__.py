"""Parts that layers are put together from.  Importing the package registers the built-in kinds."""
from . import attention, block, embedding, feed_forward, norm, position  # noqa: F401
from .base import (Block, CacheView, FeedForward, Mixer, Norm, Part, Product, Runtime, Segment, StepContext,
                   StepPlanner, Workspace)
from .registry import (
    BLOCKS,
    EMBEDDINGS,
    FEED_FORWARDS,
    HEADS,
    MIXERS,
    NORMS,
    POSITIONS,
    register_block,
    register_feed_forward,
    register_mixer,
    register_norm,
    register_position,
)
from .spec import (CacheNeed, LayerSpec, ModelSpec, PagedKVNeed, PagedNeed, ParamSpec, PartSpec, RunEntry,
                   StateNeed)
