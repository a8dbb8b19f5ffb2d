"""inference/kv_cache.py of the reference's GPU package."""
from polarquant_kv.inference.kv_cache import KVCacheManager  # noqa: F401
