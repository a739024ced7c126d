"""CPU oracle for the W4A16 matmul path -- TEST INFRASTRUCTURE ONLY.

ctypes/numpy front end of ``lane_oracle.c`` (a C restatement of the reference's CPU
algorithm; every C function cites the reference file:line it follows).  Only ``tests/``,
``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may import this
package; the product package ``llm170_b200`` never does.

Parity pin: the reference (Rust) cannot be built where this oracle was written; the
oracle is pinned by the reference's own known-answer tests, restated in
``tests/test_oracle_kat.py``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liblane_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile ``lane_oracle.c`` with gcc (see the Makefile beside it)."""
    src = os.path.join(_HERE, "lane_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "-B", "liblane_oracle.so"])
    return _SO


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = ctypes.CDLL(_SO)
        c = ctypes
        vp = c.c_void_p
        L.orc_half_to_f32.restype = c.c_float
        L.orc_half_to_f32.argtypes = [c.c_uint16]
        L.orc_bf16_to_f32.restype = c.c_float
        L.orc_bf16_to_f32.argtypes = [c.c_uint16]
        L.orc_f32_to_f16.restype = c.c_uint16
        L.orc_f32_to_f16.argtypes = [c.c_float]
        L.orc_tree64.restype = c.c_double
        L.orc_tree64.argtypes = [vp]
        L.orc_lane_parts_scale.restype = c.c_int
        L.orc_lane_parts_scale.argtypes = [vp, vp, vp, vp, c.c_int, c.c_int, vp]
        L.orc_dot_row_w4a16_lane_group.restype = c.c_float
        L.orc_dot_row_w4a16_lane_group.argtypes = [vp, vp, vp, vp, c.c_int, c.c_int]
        L.orc_dot_row_w4a16_lane.restype = c.c_float
        L.orc_dot_row_w4a16_lane.argtypes = [vp, vp, vp, vp, c.c_int]
        L.orc_dequant_row_w4a16_split.restype = None
        L.orc_dequant_row_w4a16_split.argtypes = [vp, vp, c.c_size_t, c.c_int, c.c_int, c.c_int, vp]
        L.orc_dequant_w4a16.restype = None
        L.orc_dequant_w4a16.argtypes = [vp, vp, c.c_int, c.c_int, c.c_int, c.c_int, vp]
        L.orc_marlin_repack_q.restype = c.c_int
        L.orc_marlin_repack_q.argtypes = [vp, c.c_size_t, c.c_int, c.c_int, vp]
        L.orc_marlin_unrepack_q.restype = c.c_int
        L.orc_marlin_unrepack_q.argtypes = [vp, c.c_int, c.c_int, vp]
        L.orc_marlin_permute_scales.restype = c.c_int
        L.orc_marlin_permute_scales.argtypes = [vp, c.c_size_t, c.c_int, c.c_int, c.c_int, vp]
        L.orc_select_topk.restype = c.c_int
        L.orc_select_topk.argtypes = [vp, c.c_int, c.c_int, vp, vp]
        L.orc_linear_lane_rows.restype = c.c_int
        L.orc_linear_lane_rows.argtypes = [vp, vp, vp, vp] + [c.c_int] * 8
        L.orc_linear_lane.restype = c.c_int
        L.orc_linear_lane.argtypes = [vp, vp, vp, vp] + [c.c_int] * 6
        L.orc_head_quant.restype = c.c_int
        L.orc_head_quant.argtypes = [vp, c.c_int, c.c_int, vp, vp]
        L.orc_head_gemv_i8.restype = c.c_int
        L.orc_head_gemv_i8.argtypes = [vp, vp, vp, vp, c.c_int, c.c_int, c.c_int]
        _lib = L
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dt) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dt)


def half_to_f32(h: int) -> float:
    return float(lib().orc_half_to_f32(int(h) & 0xFFFF))


def bf16_to_f32(h: int) -> float:
    return float(lib().orc_bf16_to_f32(int(h) & 0xFFFF))


def f32_to_f16(v: float) -> int:
    return int(lib().orc_f32_to_f16(float(np.float32(v))))


def tree64(v) -> float:
    a = _c(v, np.float64)
    assert a.size == 64
    return float(lib().orc_tree64(_p(a)))


def lane_parts_scale(qrow, zrow, scale_f32, x, group: int) -> np.ndarray:
    qrow, zrow = _c(qrow, np.uint32), _c(zrow, np.uint32)
    sc, x = _c(scale_f32, np.float32), _c(x, np.uint16)
    k = x.size
    if qrow.size != k // 8 or zrow.size != k // group or sc.size != k // group:
        raise ValueError("w4a16 lane: row length contract")
    out = np.zeros(64, np.float64)
    if lib().orc_lane_parts_scale(_p(qrow), _p(zrow), _p(sc), _p(x), k, group, _p(out)) != 0:
        raise ValueError(f"w4a16 lane: k must be group-aligned (group={group} k={k})")
    return out


def dot_row_w4a16_lane_group(qrow, zrow, srow_f32, x, group: int) -> np.float32:
    return np.float32(tree64(lane_parts_scale(qrow, zrow, srow_f32, x, group)))


def dot_row_w4a16_lane(qrow, zrow, srow_u16, x) -> np.float32:
    qrow, zrow = _c(qrow, np.uint32), _c(zrow, np.uint32)
    srow, x = _c(srow_u16, np.uint16), _c(x, np.uint16)
    k = x.size
    if k % 128 or qrow.size != k // 8 or srow.size != k // 128 or zrow.size != k // 128:
        raise ValueError("w4a16 lane: g128 row contract")
    return np.float32(lib().orc_dot_row_w4a16_lane(_p(qrow), _p(zrow), _p(srow), _p(x), k))


def dequant_row_w4a16_split(q_bytes, s_bytes, row: int, k: int, group: int, scale_bf16: bool):
    q, s = _c(q_bytes, np.uint8), _c(s_bytes, np.uint8)
    out = np.empty(k, np.float32)
    lib().orc_dequant_row_w4a16_split(_p(q), _p(s), row, k, group, int(scale_bf16), _p(out))
    return out


def dequant_w4a16(q_u32, s_u16, n: int, k: int, group: int, scale_bf16: bool = False):
    """f32 [n,k] = (nibble-8)*scale for every element (row function applied to all rows)."""
    q = _c(q_u32, np.uint32).reshape(n, k // 8)
    s = _c(s_u16, np.uint16).reshape(n, k // group)
    out = np.empty((n, k), np.float32)
    lib().orc_dequant_w4a16(_p(q), _p(s), n, k, group, int(scale_bf16), _p(out))
    return out


def marlin_repack_q(q_u32, n: int, k: int) -> np.ndarray:
    q = _c(q_u32, np.uint32).ravel()
    out = np.zeros((k // 16) * (n // 64) * 128 if (k % 16 == 0 and n % 64 == 0) else 1, np.uint32)
    if lib().orc_marlin_repack_q(_p(q), q.size, n, k, _p(out)) != 0:
        raise ValueError(f"marlin repack: k={k}%16 / n={n}%64 / length contract")
    return out


def marlin_unrepack_q(packed, n: int, k: int) -> np.ndarray:
    p = _c(packed, np.uint32).ravel()
    q = np.zeros(n * (k // 8), np.uint32)
    if lib().orc_marlin_unrepack_q(_p(p), n, k, _p(q)) != 0:
        raise ValueError("marlin unrepack: contract")
    return q


def marlin_permute_scales(s_f32, n: int, k: int, gs: int) -> np.ndarray:
    s = _c(s_f32, np.float32).ravel()
    out = np.zeros(max(1, (k // gs) * n), np.float32)
    if lib().orc_marlin_permute_scales(_p(s), s.size, n, k, gs, _p(out)) != 0:
        raise ValueError("marlin scales: contract")
    return out


def select_topk(logits, k: int):
    lg = _c(logits, np.float32).ravel()
    kk = min(k, lg.size)
    idx = np.zeros(max(kk, 1), np.int32)
    w = np.zeros(max(kk, 1), np.float32)
    if kk == 0:
        return []
    r = lib().orc_select_topk(_p(lg), lg.size, k, _p(idx), _p(w))
    return [(int(idx[i]), np.float32(w[i])) for i in range(r)]


def linear_lane(q_u32, s_u16, x_u16, m: int, n: int, k: int, group: int,
                scale_bf16: bool = False, nthreads: int = 0, rows=None) -> np.ndarray:
    """f32 [m,n]: every output is the reference lane dot with zero point 8.

    ``rows=(r0,r1)`` restricts the computation to those weight rows (others stay 0).
    """
    q = _c(q_u32, np.uint32).reshape(n, k // 8)
    s = _c(s_u16, np.uint16).reshape(n, k // group)
    x = _c(x_u16, np.uint16).reshape(m, k)
    out = np.zeros((m, n), np.float32)
    if nthreads <= 0:
        nthreads = os.cpu_count() or 1
    r0, r1 = (0, n) if rows is None else rows
    rc = lib().orc_linear_lane_rows(_p(q), _p(s), _p(x), _p(out), m, n, k, group,
                                    int(scale_bf16), r0, r1, nthreads)
    if rc != 0:
        raise ValueError("linear_lane: shape contract")
    return out


def moe_ffn(x_u16, logits, w13_q, w13_s, w2_q, w2_s, top_k: int, group: int, experts=None) -> np.ndarray:
    """CPU restatement of the resident MoE FFN: routing by select_topk
    (crates/core/src/qwen35/stages/moe.rs:8-31); per expert the two linears are lane dots; the rounding
    points follow the reference's GPU path (crates/backend-gpu/src/rawcuda/w4a16_dec/kernels/marlin_moe.rs:290-422):
    c13 -> f16, silu(g)*u -> f16 (crates/backend-gpu/src/rawcuda/assets/moe.cu:1649-1660), f16(c2) * f16(w) -> f16
    (the epilogue of the grouped GEMM, crates/backend-gpu/src/rawcuda/assets/marlin_moe/marlin_template.h:1515-1524),
    then the f32 sum over k in rank order (crates/backend-gpu/src/rawcuda/assets/moe.cu:1662-1674).
    `experts=(e0,e1)` keeps only that range (one rank's share under expert parallelism)."""
    x = _c(x_u16, np.uint16)
    t, h = x.shape
    n_exp, f2, _ = w13_q.shape
    f = f2 // 2
    lg = _c(logits, np.float32).reshape(t, n_exp)
    sel = [select_topk(lg[i], top_k) for i in range(t)]
    e0, e1 = (0, n_exp) if experts is None else experts
    contrib = np.zeros((t, top_k, h), np.float32)
    for e in range(e0, e1):
        rows = [(i, r, w) for i in range(t) for r, (ee, w) in enumerate(sel[i]) if ee == e]
        if not rows:
            continue
        xs = np.ascontiguousarray(x[[i for i, _, _ in rows]])
        c13 = linear_lane(w13_q[e], w13_s[e], xs, len(rows), 2 * f, h, group).astype(np.float16).astype(np.float32)
        g, u = c13[:, :f], c13[:, f:]
        act = ((g / (np.float32(1.0) + np.exp(-g, dtype=np.float32))) * u).astype(np.float16)
        c2 = linear_lane(w2_q[e], w2_s[e], act.view(np.uint16), len(rows), h, f, group)
        # marlin_moe/marlin_template.h:1515-1524: the f16 result times the f16-rounded routing weight, rounded to f16
        wv = np.array([w for _, _, w in rows], np.float32)[:, None].astype(np.float16).astype(np.float32)
        c2 = (c2.astype(np.float16).astype(np.float32) * wv).astype(np.float16).astype(np.float32)
        for j, (i, r, _) in enumerate(rows):
            contrib[i, r] = c2[j]
    out = np.zeros((t, h), np.float32)
    for r in range(top_k):
        out = out + contrib[:, r]
    return out


def head_quant(w_bf16, n: int, k: int):
    """crates/backend-gpu/src/rawcuda/w4a16_dec/upload.rs:1472-1518: per-row int8 quantisation of the bf16 lm-head
    (scale = absmax/127, round half away from zero).  Returns (q int8 [n,k], scale f32 [n])."""
    w = _c(w_bf16, np.uint16).reshape(n, k)
    q = np.zeros((n, k), np.int8)
    sc = np.zeros(n, np.float32)
    if lib().orc_head_quant(_p(w), n, k, _p(q), _p(sc)) != 0:
        raise ValueError("head_quant: bad shape")
    return q, sc


def head_gemv_i8(q, scale, x32, t: int) -> np.ndarray:
    """crates/backend-gpu/src/rawcuda/assets/head.cu:100-225 (64 lanes, un-fused f32 products, f64 tree):
    out f32 [t,n] = (q @ x^T) * scale."""
    q = _c(q, np.int8)
    n, k = q.shape
    x = _c(x32, np.float32).reshape(t, k)
    sc = _c(scale, np.float32)
    out = np.zeros((t, n), np.float32)
    if lib().orc_head_gemv_i8(_p(q), _p(sc), _p(x), _p(out), n, k, t) != 0:
        raise ValueError("head_gemv_i8: bad shape")
    return out
