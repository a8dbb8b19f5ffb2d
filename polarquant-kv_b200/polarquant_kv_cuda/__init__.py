"""Module paths of the reference's GPU package (src/polarquant_kv_cuda/) over this library.

Code written against ``polarquant_kv_cuda`` imports ``compress_kernel.compress_gpu``,
``decompress_kernel.decompress_gpu``, ``attention_kernel.compressed_attention_gpu``, ``qjl_kernel.*``,
``rotation``, ``lloyd_max``, ``types.CompressedKVCacheGPU``, ``compressor`` and ``inference.*``.  Every module
here is a thin binding of those names to ``polarquant_kv``: the functions run the sm_100a kernels through the
C ABI and keep the reference's argument order; caches are block_pq4 (``polarquant_kv.types.CompressedKV``)."""
