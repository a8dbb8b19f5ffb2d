"""rotation.py:8-30 of the reference's GPU package: the matrix as a float32 tensor on the device."""
import torch

from polarquant_kv import rotation as _r


def generate_rotation_matrix(d: int, seed: int | None = None, device="cuda") -> torch.Tensor:
    return torch.from_numpy(_r.generate_rotation_matrix(d, seed)).to(device=device, dtype=torch.float32)


def rotate(v: torch.Tensor, R: torch.Tensor) -> torch.Tensor:
    """v @ R^T in float32, returned in v's dtype."""
    return (v.float() @ R.float().T).to(v.dtype)


def inverse_rotate(v: torch.Tensor, R: torch.Tensor) -> torch.Tensor:
    """v @ R in float32, returned in v's dtype."""
    return (v.float() @ R.float()).to(v.dtype)
