"""compress_kernel.py:100-189 of the reference's GPU package."""
from polarquant_kv.quantizer import compress as _compress


def compress_gpu(kv, rotation_matrix, n_bits: int = 4, group_size: int = 32, jl_matrix=None):
    """kv [batch, heads, seq, head_dim] float16 on the GPU -> compressed cache (pq_compress_rows)."""
    return _compress(kv, rotation_matrix, n_bits, group_size, jl_matrix)
