"""polarquant_kv — B200 (sm_100a) implementation of the PolarQuant-KV block_pq4 hot path.

Module and function names follow hilllief/polarquant-kv (``python/polarquant_kv`` and the
GPU facade ``src/polarquant_kv_cuda/compressor.py``); tensors are torch CUDA tensors and
every hot operation runs in hand-written CUDA kernels behind a C ABI
(``libpolarquant_b200.so``, declared in ``include/polarquant_b200.h``).  There is no CPU
or eager-PyTorch fallback: if the library has not been built, importing ``_ext`` raises.
"""

__version__ = "0.1.0"
