"""Seeded orthogonal rotation (python/polarquant_kv/rotation.py of the reference) and the
device-side forms of it the kernels consume."""

from __future__ import annotations

import hashlib

import numpy as np
import torch
from scipy.stats import ortho_group

ROT_SCALE = 4096.0   # power of two applied before the float16 split of R
JL_SCALE = 1024.0    # same for the folded JL matrix P @ R^T


def generate_rotation_matrix(d: int, seed: int | None = None) -> np.ndarray:
    """d x d Haar-distributed orthogonal matrix, float64 — the same draw as the reference
    (scipy.stats.ortho_group with numpy.random.default_rng(seed); rotation.py:7-35),
    including its d == 1 special case and its ValueError on a bad d."""
    if not isinstance(d, (int, np.integer)):
        raise ValueError(f"d must be an integer, got {type(d).__name__}")
    if d <= 0:
        raise ValueError(f"d must be a positive integer, got {d}")
    if d == 1:
        rng = np.random.Generator(np.random.PCG64(seed))
        return np.array([[rng.choice([-1.0, 1.0])]], dtype=np.float64)
    return ortho_group.rvs(d, random_state=np.random.default_rng(seed)).astype(np.float64)


def rotate(v, rotation_matrix):
    """v @ R^T in float64, cast back to v's dtype (rotation.py:38-48).  numpy or torch."""
    if isinstance(v, torch.Tensor):
        R = torch.as_tensor(np.asarray(rotation_matrix, dtype=np.float64) if not isinstance(
            rotation_matrix, torch.Tensor) else rotation_matrix, device=v.device).double()
        return (v.double() @ R.T).to(v.dtype)
    return (v.astype(np.float64) @ np.asarray(rotation_matrix).T).astype(v.dtype)


def inverse_rotate(v, rotation_matrix):
    """v @ R in float64, cast back to v's dtype (rotation.py:51-61).  numpy or torch."""
    if isinstance(v, torch.Tensor):
        R = torch.as_tensor(np.asarray(rotation_matrix, dtype=np.float64) if not isinstance(
            rotation_matrix, torch.Tensor) else rotation_matrix, device=v.device).double()
        return (v.double() @ R).to(v.dtype)
    return (v.astype(np.float64) @ np.asarray(rotation_matrix)).astype(v.dtype)


def split_fp16(m: np.ndarray, scale: float) -> np.ndarray:
    """[rows, cols] float64 -> float16 [rows, 2*cols] = [hi | lo] with
    scale*m ~= hi + lo (two-term split, about 22 significant bits)."""
    s = np.asarray(m, dtype=np.float64) * scale
    hi = s.astype(np.float16)
    lo = (s - hi.astype(np.float64)).astype(np.float16)
    return np.concatenate([hi, lo], axis=1)


def _as_numpy64(m) -> np.ndarray:
    if isinstance(m, torch.Tensor):
        return m.detach().double().cpu().numpy()
    return np.asarray(m, dtype=np.float64)


class DevicePlan:
    """Device-resident constants derived from a rotation (and optionally a JL) matrix:
    float32 R for the attention kernels, the float16 split of R for compress, float32 P and
    the split of P @ R^T for the QJL sketch.  Built once and cached by content."""

    def __init__(self, rotation_matrix, device, jl_matrix=None):
        R = _as_numpy64(rotation_matrix)
        if R.ndim != 2 or R.shape[0] != R.shape[1]:
            raise ValueError(f"rotation matrix must be square, got {R.shape}")
        self.head_dim = R.shape[0]
        self.device = torch.device(device)
        self.rot = torch.from_numpy(R.astype(np.float32)).contiguous().to(self.device)
        self.rot_split = torch.from_numpy(split_fp16(R, ROT_SCALE)).contiguous().to(self.device)
        self.jl = None
        self.jl_split = None
        self.jl_dim = 0
        if jl_matrix is not None:
            P = _as_numpy64(jl_matrix)
            if P.ndim != 2 or P.shape[1] != self.head_dim:
                raise ValueError(f"jl_matrix must be [jl_dim, {self.head_dim}], got {P.shape}")
            self.jl_dim = P.shape[0]
            self.jl = torch.from_numpy(P.astype(np.float32)).contiguous().to(self.device)
            self.jl_split = torch.from_numpy(split_fp16(P @ R.T, JL_SCALE)).contiguous().to(self.device)


_PLANS: dict = {}


def _digest(m) -> str:
    if m is None:
        return "-"
    a = _as_numpy64(m)
    return hashlib.blake2b(a.tobytes(), digest_size=16).hexdigest() + str(a.shape)


_QUICK: dict = {}
_QUICK_LIMIT = 64


def _quick_key(m):
    """Identity of a matrix object without reading it: the object, where its data lives and, for arrays,
    three probe values (for tensors the version counter) - enough to notice the in-place edits that the
    content digest would notice, at no cost per call.  None when the object offers no such handle."""
    if m is None:
        return ("-",)
    if isinstance(m, np.ndarray):
        if m.size == 0:
            return None
        flat = m.reshape(-1) if m.flags.c_contiguous else None
        if flat is None:
            return None
        return ("np", id(m), m.shape, m.dtype.str, m.ctypes.data, float(flat[0]), float(flat[m.size // 2]), float(flat[-1]))
    if isinstance(m, torch.Tensor):
        return ("pt", id(m), tuple(m.shape), str(m.dtype), m.data_ptr(), m._version)
    return None


def device_plan(rotation_matrix, device, jl_matrix=None) -> DevicePlan:
    """Cached DevicePlan for (R, P, device).  The same matrix OBJECTS are recognised without being read
    (the usual case: a caller passes its R and P on every call); otherwise the plan is looked up by a digest
    of the contents.  Callers on a hot loop can also hold the plan and pass it instead of R."""
    if isinstance(rotation_matrix, DevicePlan):
        return rotation_matrix
    dev = str(torch.device(device))
    qr, qp = _quick_key(rotation_matrix), _quick_key(jl_matrix)
    quick = (qr, qp, dev) if qr is not None and qp is not None else None
    if quick is not None:
        hit = _QUICK.get(quick)
        if hit is not None:
            return hit[0]
    key = (_digest(rotation_matrix), _digest(jl_matrix), dev)
    plan = _PLANS.get(key)
    if plan is None:
        plan = DevicePlan(rotation_matrix, device, jl_matrix)
        _PLANS[key] = plan
    if quick is not None:
        if len(_QUICK) >= _QUICK_LIMIT:
            _QUICK.pop(next(iter(_QUICK)))
        _QUICK[quick] = (plan, rotation_matrix, jl_matrix)      # the references keep the ids from being reused
    return plan
