from .manager import (  # noqa: F401
    BlockTable,
    CacheError,
    CacheManager,
    IdPool,
    KVGroupSpec,
    RequestCache,
    group_caches,
)
