"""qjl_kernel.py:6-135 of the reference's GPU package."""
import torch

from polarquant_kv.qjl import bit_pack, bit_unpack, compute_correction, compute_signatures  # noqa: F401


def compute_signatures_gpu(residual: torch.Tensor, jl_matrix) -> tuple[torch.Tensor, torch.Tensor]:
    """residual [..., d] -> (packed sign bits uint8 [..., jl_dim / 8], residual norms float16 [...])."""
    sig = compute_signatures(residual, jl_matrix)
    norms = sig.residual_norm
    if not isinstance(norms, torch.Tensor):
        norms = torch.tensor(norms, device=residual.device)
    return bit_pack(sig.signs), norms.to(torch.float16)


def compute_correction_gpu(query, packed_signs, residual_norms, jl_matrix) -> torch.Tensor:
    return compute_correction(query, packed_signs, residual_norms, jl_matrix)
