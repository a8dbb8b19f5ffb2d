"""decompress_kernel.py:10-51 of the reference's GPU package."""
import torch

from polarquant_kv.quantizer import decompress as _decompress


def decompress_gpu(cache, rotation_matrix) -> torch.Tensor:
    """Compressed cache -> [batch, heads, seq, head_dim] float16 (pq_dequant)."""
    return _decompress(cache, rotation_matrix, torch.float16)
