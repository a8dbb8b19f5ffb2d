"""attention_kernel.py:11-113 of the reference's GPU package."""
from polarquant_kv.attention import compressed_attention as _attention


def compressed_attention_gpu(query, compressed_keys, compressed_values, rotation_matrix, jl_matrix=None,
                             enable_qjl: bool = True, num_kv_heads: int | None = None):
    """query [batch, q_heads, seq_q, head_dim] float16 over compressed caches (fused decode / prefill kernels)."""
    return _attention(query, compressed_keys, compressed_values, rotation_matrix, jl_matrix, enable_qjl, num_kv_heads)
