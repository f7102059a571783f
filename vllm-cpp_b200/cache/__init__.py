from .device_cache import CacheGroup, CacheLayout, DeviceCache, KVCacheView, StateCacheView

__all__ = ["CacheGroup", "CacheLayout", "DeviceCache", "KVCacheView", "StateCacheView"]
