from .block_cache import CacheBlock
from .kvcache_manager import KVCacheManager, RPCKVCacheManager
from .state_cache import StateCacheManager

__all__ = ["CacheBlock", "KVCacheManager", "RPCKVCacheManager", "StateCacheManager"]
