"""types.py:8-21 of the reference's GPU package; the cache container is the block_pq4 one."""
from polarquant_kv.types import CompressedKV as CompressedKVCacheGPU  # noqa: F401
from polarquant_kv.types import CompressedKV, QJLSignatures  # noqa: F401
