from .cache_manager import CacheManager, get_cache_manager, reset_cache_manager

__all__ = ["CacheManager", "get_cache_manager", "reset_cache_manager"]
