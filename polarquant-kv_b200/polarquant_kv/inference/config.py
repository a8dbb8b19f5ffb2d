"""Configuration of the compressed cache (src/polarquant_kv_cuda/inference/config.py:6-12 of the
reference, plus an independent bit width for the values)."""

from dataclasses import dataclass


@dataclass
class PolarQuantConfig:
    n_bits: int = 4                 # key indices (and value indices unless v_bits is given)
    group_size: int = 32
    jl_dim: int = 64
    enable_qjl: bool = False
    enable_compression: bool = True
    v_bits: int | None = None
