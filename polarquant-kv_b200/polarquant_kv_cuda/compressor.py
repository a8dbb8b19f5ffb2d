"""compressor.py:11-38 of the reference's GPU package."""
from polarquant_kv.compressor import compress, compressed_attention, decompress, get_memory_bytes  # noqa: F401
