"""Mirror of the reference's standalone ``Gptq4`` parity-gate entry
(crates/backend-gpu/src/rawcuda/gptq4.rs): host slices in, f32 out."""
from __future__ import annotations

import numpy as np

from . import _lib
from .w4a16_dec import W4a16Dec, W4a16Error


def check_shapes(t: int, qlen: int, slen: int, xlen: int, n: int, k: int, group: int) -> None:
    """gptq4.rs:31-58 (lengths in elements).  Raises on a violated contract.

    The reference additionally caps k at group*256 for t == 1 because its GEMV keeps a row's
    scales in shared memory (gptq4.rs:51-56); this implementation has no such limit.
    """
    if min(t, qlen, slen, xlen, n, k, group) < 0 or \
            _lib.lib().w4a16_check_shapes(t, qlen, slen, xlen, n, k, group) != 0:
        raise W4a16Error(f"gptq4: shape contract violated q={qlen} s={slen} x={xlen} n={n} k={k} t={t} group={group}")


def kernel_sym(gemm: bool, group: int, scale_bf16: bool) -> str:
    """gptq4.rs:60-70: which kernel family serves a (group, scale type) combination -- here the template
    instantiations of csrc/gemm_tc.cu (t > 8) and csrc/gemv_sk.cu (decode), as `W4a16Dec.last_kernel` reports them."""
    if group not in (128, 64, 32):
        raise W4a16Error(f"gptq4: unsupported combination group={group} scale_bf16={scale_bf16}")
    g = 32 if group == 64 else group      # group 64 is stored as two groups of 32 with the same scale
    return f"gemm_w4a16_tc_kernel<{g},1>" if gemm else f"gemv_sk_kernel<{g},true>"


class Gptq4:
    def __init__(self, device: int = 0):
        self.dec = W4a16Dec(device)

    def gemv(self, x, q, s, n, k, group, scale_bf16=False):
        return self.gemm(x, 1, q, s, n, k, group, scale_bf16)

    def gemm(self, x, t, q, s, n, k, group, scale_bf16=False) -> np.ndarray:
        x = np.ascontiguousarray(x).view(np.uint16).ravel()
        q = np.ascontiguousarray(q).view(np.uint32).ravel()
        s = np.ascontiguousarray(s).view(np.uint16).ravel()
        check_shapes(t, q.size, s.size, x.size, n, k, group)
        out = np.empty((t, n), np.float32)
        d = self.dec
        d._ck(d._L.w4a16_gptq4_gemm(d._h, x.ctypes.data, t, q.ctypes.data, s.ctypes.data, n, k, group,
                                    int(scale_bf16), out.ctypes.data))
        return out
