"""Builds libpolarquant_b200.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m polarquant_kv._build            # from the polarquant-kv_b200 directory

The library lands beside this file so it travels with the source tree; nothing is
installed into site-packages and no JIT cache is used.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(PKG_DIR), "csrc")
INCLUDE = os.path.join(os.path.dirname(os.path.dirname(PKG_DIR)), "include")
LIB_PATH = os.path.join(PKG_DIR, "libpolarquant_b200.so")

SOURCES = ["pq_compress.cu", "pq_dequant.cu", "pq_decode_attn.cu", "pq_prefill_attn.cu", "pq_lse_merge.cu", "pq_qjl.cu",
           "pq_llama_abi.cu"]
HEADERS = ["pq_common.cuh", "pq_tcgen05.cuh", os.path.join(INCLUDE, "polarquant_b200.h"),
           os.path.join(INCLUDE, "polarquant_llama_abi.h")]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put /usr/local/cuda/bin on PATH")


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, s) for s in SOURCES] + [h if os.path.isabs(h) else os.path.join(CSRC, h) for h in HEADERS]
    return any(os.path.getmtime(d) > built for d in deps if os.path.exists(d))


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile every kernel for sm_100a and link the shared library; returns its path."""
    if not force and not _stale():
        return LIB_PATH
    nvcc = _nvcc()
    objs = []
    build_dir = os.path.join(CSRC, "build")
    os.makedirs(build_dir, exist_ok=True)
    common = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-I", INCLUDE, "-I", CSRC]
    if verbose:
        common += ["-Xptxas", "-v"]
    common += os.environ.get("PQ_NVCC_FLAGS", "").split()     # extra flags for experiments
    procs = []
    for src in SOURCES:
        path = os.path.join(CSRC, src)
        if not os.path.exists(path):
            continue
        obj = os.path.join(build_dir, src.replace(".cu", ".o"))
        objs.append(obj)
        procs.append((src, subprocess.Popen(common + ["-c", path, "-o", obj], stdout=subprocess.PIPE,
                                            stderr=subprocess.STDOUT, text=True)))
    for src, proc in procs:
        out, _ = proc.communicate()
        if verbose and out:
            print(out)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out}")
    link = [nvcc, "-shared", "-o", LIB_PATH] + objs + ["-lcudart"]
    res = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}")
    return LIB_PATH


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
