"""lloyd_max.py:12-110 of the reference's GPU package."""
import numpy as np
import torch

from polarquant_kv.codebook import build_lloyd_max_codebook, dequantize_with_codebook, quantize_with_codebook  # noqa: F401


def get_codebook_torch(dim: int, n_bits: int, device="cuda") -> torch.Tensor:
    centroids = build_lloyd_max_codebook(dim, n_bits)
    centroids = centroids[0] if isinstance(centroids, tuple) else centroids
    return torch.from_numpy(np.asarray(centroids, dtype=np.float32)).to(device)
