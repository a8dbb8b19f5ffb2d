"""utils.py of the reference's GPU package."""
from polarquant_kv.utils import *  # noqa: F401,F403
from polarquant_kv.utils import check_memory_warning, cosine_similarity, estimate_memory_bytes  # noqa: F401


def cosine_similarity_gpu(a, b) -> float:
    """Cosine similarity of two tensors, flattened, in float32 (utils.py:6-10)."""
    import torch
    return torch.nn.functional.cosine_similarity(a.flatten().float(), b.flatten().float(), dim=0).item()
