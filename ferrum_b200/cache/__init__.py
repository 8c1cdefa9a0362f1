from .storage import CacheLayout, CacheStorage, LayerCache

__all__ = ["CacheLayout", "CacheStorage", "LayerCache"]
