"""Generates the committed fixtures in this directory by running the REFERENCE's own
Python functions (hilllief/polarquant-kv), imported from a checkout given on the command
line.  The reference is not redistributed and is not needed to run the tests; this
script documents exactly how every fixture was produced.

    python tests/golden/make_golden.py /path/to/polarquant-kv

block_pq4 is produced by composing reference calls only:
    polarquant_kv.rotation.generate_rotation_matrix / rotate / inverse_rotate
    polarquant_kv_cuda.lloyd_max.build_lloyd_max_codebook / quantize_with_codebook /
        dequantize_with_codebook
    polarquant_kv_cuda.compress_kernel._bit_pack_quantized
    polarquant_kv.qjl.generate_jl_matrix (+ compute_signatures / compute_correction via
        the unmodified polarquant_kv.attention.compressed_attention, whose module-level
        names ``compress`` / ``decompress`` are rebound to the block_pq4 codec)
The per-block float32 radius is numpy's ``np.linalg.norm(blocks, axis=-1)``.
Inputs come from oracle/inputs.py (seeded); their sha256 is stored beside the outputs.
"""

from __future__ import annotations

import os
import sys
from dataclasses import dataclass

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)


def load_reference(path: str):
    sys.path.insert(0, os.path.join(path, "python"))
    sys.path.insert(0, os.path.join(path, "src"))
    import polarquant_kv.attention as ref_attention
    import polarquant_kv.qjl as ref_qjl
    import polarquant_kv.rotation as ref_rotation
    import polarquant_kv_cuda.compress_kernel as ref_pack
    import polarquant_kv_cuda.lloyd_max as ref_lm
    return ref_rotation, ref_lm, ref_pack, ref_qjl, ref_attention


@dataclass
class Coded:
    d16: np.ndarray
    idx: np.ndarray


class RefCodec:
    """block_pq4 built from reference calls, one vector at a time (as the reference does)."""

    def __init__(self, ref, n_bits: int):
        self.rot, self.lm, self.pack, _, _ = ref
        self.n_bits = n_bits
        self.codebook, _ = self.lm.build_lloyd_max_codebook(32, n_bits)

    def compress(self, v, R, n_bits=None, group_size=None) -> Coded:
        xr = self.rot.rotate(v.astype(np.float32), R)
        blk = xr.reshape(-1, 32)
        d32 = np.linalg.norm(blk, axis=-1).astype(np.float32)
        zero = d32 < 1e-30
        safe = np.where(zero, np.float32(1), d32).astype(np.float32)
        direction = (blk / safe[:, None]).astype(np.float32)
        idx = self.lm.quantize_with_codebook(direction, self.codebook)
        idx[zero] = 0
        d32 = np.where(zero, np.float32(0), d32)
        # radius clamp to the float16 range as in compress_kernel.py:178
        return Coded(d16=np.minimum(d32, np.float32(65504.0)).astype(np.float16), idx=idx.reshape(-1))

    def decompress(self, c: Coded, R) -> np.ndarray:
        vals = self.lm.dequantize_with_codebook(c.idx, self.codebook).reshape(-1, 32)
        vals = (vals * c.d16.astype(np.float32)[:, None]).astype(np.float32).reshape(-1)
        return self.rot.inverse_rotate(vals, R).astype(np.float32)

    def blocks(self, c: Coded) -> np.ndarray:
        import torch
        packed = self.pack._bit_pack_quantized(
            torch.from_numpy(c.idx.reshape(-1, 32).copy()), self.n_bits).numpy()
        out = np.empty((packed.shape[0], 2 + packed.shape[1]), dtype=np.uint8)
        out[:, :2] = c.d16.astype("<f2").view(np.uint8).reshape(-1, 2)
        out[:, 2:] = packed
        return out


def encode_tensor(codec: RefCodec, x: np.ndarray, R) -> np.ndarray:
    lead = x.shape[:-1]
    flat = x.reshape(-1, x.shape[-1])
    out = [codec.blocks(codec.compress(flat[i], R)) for i in range(flat.shape[0])]
    return np.stack(out).reshape(lead + out[0].shape)


def ref_attention_call(ref, codec_k, codec_v, q, K, V, R, P, enable_qjl):
    """Unmodified reference compressed_attention with compress/decompress rebound.
    K uses codec_k and V codec_v: the reference compresses the key first and the value
    second for every token (attention.py:138-144), so the calls alternate."""
    att = ref[4]
    state = {"n": 0}

    def compress(v, R_, n_bits, group_size):
        codec = codec_k if state["n"] % 2 == 0 else codec_v
        state["n"] += 1
        c = codec.compress(v, R_)
        c.codec = codec
        return c

    def decompress(c, R_):
        return c.codec.decompress(c, R_)

    saved = att.compress, att.decompress
    att.compress, att.decompress = compress, decompress
    try:
        return att.compressed_attention(q, K, V, R, jl_matrix=P, n_bits=4, group_size=32,
                                        enable_qjl=enable_qjl, num_kv_heads=K.shape[0])
    finally:
        att.compress, att.decompress = saved


def main(ref_path: str) -> None:
    from oracle import inputs

    ref = load_reference(ref_path)
    rot, lm, _, qjl, _ = ref
    out = {}

    for bits in (2, 4):
        c, b = lm.build_lloyd_max_codebook(32, bits)
        out[f"codebook_dim32_b{bits}"] = c
        out[f"boundaries_dim32_b{bits}"] = b
    for d in (64, 128):
        out[f"R_d{d}_seed0"] = rot.generate_rotation_matrix(d, 0)
    out["P_m64_d64_seed1"] = qjl.generate_jl_matrix(64, 64, 1)
    out["P_m128_d128_seed1"] = qjl.generate_jl_matrix(128, 128, 1)

    codec4, codec2 = RefCodec(ref, 4), RefCodec(ref, 2)

    # ---- case c0: the CPU-runnable configuration (D=64, 4-bit, GQA 7:1, S=512)
    K, V, q = inputs.make_kvq(**inputs.C0)
    R = out["R_d64_seed0"]
    P = out["P_m64_d64_seed1"]
    out["c0_input_sha256"] = np.array(inputs.digest(K, V, q))
    out["c0_k_blocks_b4"] = encode_tensor(codec4, K[0], R)
    out["c0_v_blocks_b4"] = encode_tensor(codec4, V[0], R)
    out["c0_attn_b4"] = ref_attention_call(ref, codec4, codec4, q[0], K[0], V[0], R, None, False)
    out["c0_attn_b4_qjl"] = ref_attention_call(ref, codec4, codec4, q[0], K[0], V[0], R, P, True)

    # ---- case d128: small head_dim-128 tensors, 4-bit, 2-bit, mixed K4/V2, QJL m=128
    cfg = dict(batch=1, kv_heads=2, q_heads=8, seq=96, head_dim=128, seed=3)
    K, V, q = inputs.make_kvq(**cfg)
    R = out["R_d128_seed0"]
    P = out["P_m128_d128_seed1"]
    out["d128_input_sha256"] = np.array(inputs.digest(K, V, q))
    out["d128_k_blocks_b4"] = encode_tensor(codec4, K[0], R)
    out["d128_v_blocks_b4"] = encode_tensor(codec4, V[0], R)
    out["d128_k_blocks_b2"] = encode_tensor(codec2, K[0], R)
    out["d128_v_blocks_b2"] = encode_tensor(codec2, V[0], R)
    out["d128_attn_b4"] = ref_attention_call(ref, codec4, codec4, q[0], K[0], V[0], R, None, False)
    out["d128_attn_b4_qjl"] = ref_attention_call(ref, codec4, codec4, q[0], K[0], V[0], R, P, True)
    out["d128_attn_b2"] = ref_attention_call(ref, codec2, codec2, q[0], K[0], V[0], R, None, False)
    out["d128_attn_k4v2"] = ref_attention_call(ref, codec4, codec2, q[0], K[0], V[0], R, None, False)
    # QJL side band of the 4-bit keys, from the reference's own signature routine
    signs = np.zeros((2, 96, 128), dtype=bool)
    norms = np.zeros((2, 96), dtype=np.float64)
    for h in range(2):
        for s in range(96):
            c = codec4.compress(K[0, h, s], R)
            sig = qjl.compute_signatures(K[0, h, s] - codec4.decompress(c, R), P)
            signs[h, s], norms[h, s] = sig.signs, sig.residual_norm
    out["d128_qjl_signs_b4"] = np.packbits(signs.astype(np.uint8), axis=-1, bitorder="little")
    out["d128_qjl_norms_b4"] = norms

    # ---- edge vectors: zero, single spike, fp16 extremes, tiny values (D=128)
    edge = np.zeros((6, 128), dtype=np.float16)
    edge[1, 5] = 1.0
    edge[2, :] = 65504.0
    edge[3, :] = -65504.0
    edge[4, :] = 6e-8
    edge[5, ::2] = 3.0
    edge[5, 1::2] = -3.0
    out["edge_x"] = edge
    out["edge_blocks_b4"] = encode_tensor(codec4, edge, R)
    out["edge_blocks_b2"] = encode_tensor(codec2, edge, R)

    path = os.path.join(HERE, "pq4_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes;", len(out), "arrays")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path to a checkout of the reference repository>")
    main(sys.argv[1])
