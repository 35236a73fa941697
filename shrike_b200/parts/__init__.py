"""Parts a layer is put together from.  Importing the package registers the built-in ones."""

from . import attention, block, embedding, mlp, norm, rotary  # noqa: F401
from .base import (  # noqa: F401
    BLOCKS,
    EMBEDDINGS,
    HEADS,
    FEED_FORWARDS,
    MIXERS,
    NORMS,
    POSITIONS,
    KVNeed,
    ParamSpec,
    StateNeed,
    part_class,
    register_part,
)
