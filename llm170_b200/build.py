"""Builds ``libw4a16_b200.so`` in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
SO = os.path.join(HERE, "libw4a16_b200.so")
HASH = SO + ".srchash"
SOURCES = ["dec.cu", "repack.cu", "gemv.cu", "gemv_sk.cu", "gemv_rb.cu", "gemm_tc.cu", "moe.cu", "moe_host.cu", "gemv_static.cu", "loader.cu", "head.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall", "--shared", "-cudart", "static",
]


def source_hash() -> str:
    """sha256 over the CUDA sources, the public header and the compiler flags: what the binary is made from."""
    h = hashlib.sha256()
    files = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC))
    files.append(os.path.join(os.path.dirname(HERE), "include", "w4a16_b200.h"))
    for f in files:
        h.update(os.path.basename(f).encode())
        with open(f, "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS + SOURCES).encode())
    return h.hexdigest()


def _stale() -> bool:
    """The binary is current when the hash recorded beside it equals the hash of the sources (file times do not
    survive a copy of the tree to another machine; contents do)."""
    if not os.path.exists(SO) or not os.path.exists(HASH):
        return True
    with open(HASH) as fh:
        return fh.read().strip() != source_hash()


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return SO
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else [])
    cmd += [os.path.join(CSRC, s) for s in SOURCES] + ["-o", SO]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed building libw4a16_b200.so")
    with open(HASH, "w") as fh:
        fh.write(source_hash() + "\n")
    return SO


if __name__ == "__main__":
    build(force=True, verbose="-v" in sys.argv)
    print(SO)
