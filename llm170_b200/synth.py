"""Seeded synthetic W4A16 tensors (stand-ins for real checkpoints, which are not shipped).

Quantiser recipe follows the reference's fixture generator, scripts/gen_tiny_w4a16.py:28-53:
per row and per group of ``group`` input channels, ``scale = absmax/7`` stored as f16
(an all-zero group uses 1e-6/7), ``q = clamp(round_half_even(w/scale), -8, 7)``, stored as the
nibble ``q+8`` at bits ``4*(i&7)`` of little-endian word ``i>>3`` (compressed-tensors
``pack-quantized``; crates/core/src/w4a16.rs:124-175).  Weights are f32 N(0, sigma) and
activations f16 N(0, 1) (optionally scaled by 1/sqrt(K)) from ``numpy`` PCG64 streams.
"""
from __future__ import annotations

import numpy as np


def quantize_sym_int4(w: np.ndarray, group: int, scale_bf16: bool = False):
    """w f32 [n,k] -> (q u32 [n,k/8], s u16 [n,k/group]); s holds f16 bits, or bf16 bits (the f32 value
    truncated to its upper half, as the reference's generator writes them) when ``scale_bf16``."""
    n, k = w.shape
    assert k % group == 0 and k % 8 == 0
    wg = w.reshape(n, k // group, group).astype(np.float32)
    amax = np.abs(wg).max(axis=2)
    amax = np.where(amax == 0, np.float32(1e-6), amax).astype(np.float32)
    s32 = (amax / np.float32(7.0)).astype(np.float32)
    if scale_bf16:
        sbits = (s32.view(np.uint32) >> 16).astype(np.uint16)
        sf = (sbits.astype(np.uint32) << 16).view(np.float32)
    else:
        sbits = s32.astype(np.float16).view(np.uint16)
        sf = sbits.view(np.float16).astype(np.float32)
    # guard: a scale that rounds to zero would divide by zero
    sf = np.where(sf == 0, np.float32(2.0 ** -24), sf)
    qv = np.clip(np.rint(wg / sf[:, :, None]), -8, 7).astype(np.int32) + 8
    nib = qv.reshape(n, k // 8, 8).astype(np.uint32)
    shifts = (4 * np.arange(8, dtype=np.uint32))[None, None, :]
    q = np.bitwise_or.reduce(nib << shifts, axis=2).astype(np.uint32)
    return q, np.ascontiguousarray(sbits.reshape(n, k // group))


def make_linear(n: int, k: int, group: int, seed: int, sigma: float = 0.02, scale_bf16: bool = False):
    """Deterministic int4 linear: returns (q u32 [n,k/8], s u16 [n,k/group])."""
    rng = np.random.Generator(np.random.PCG64(seed))
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(sigma)
    return quantize_sym_int4(w, group, scale_bf16)


def make_acts(m: int, k: int, seed: int, scale: float = 1.0) -> np.ndarray:
    """f16 activations [m,k] as u16 bit patterns; N(0,1)*scale."""
    rng = np.random.Generator(np.random.PCG64(seed ^ 0x5EED5EED))
    x = rng.standard_normal((m, k), dtype=np.float32) * np.float32(scale)
    return x.astype(np.float16).view(np.uint16)


def make_router_logits(t: int, n_exp: int, seed: int) -> np.ndarray:
    rng = np.random.Generator(np.random.PCG64(seed ^ 0x70FFEE))
    return rng.standard_normal((t, n_exp), dtype=np.float32)


# 27B-class dense decoder linears (K, N) named as the reference names its call sites.
DENSE_27B = {
    "gate_up": (5120, 34816),
    "down": (17408, 5120),
    "qkv": (5120, 7168),
    "o_proj": (6144, 5120),
}

# lm-head of the same 27B-class decoder: (vocabulary rows, hidden).
LM_HEAD_27B = (151936, 5120)

# 35B-A3B-class MoE layer.
MOE_35B = {"n_experts": 128, "hidden": 2048, "moe_ffn": 768, "top_k": 8, "group": 32}


def decode_bytes(n: int, k: int, m: int, group: int = 128) -> int:
    """Algorithmic bytes of one W4A16 linear call: int4 weights + f16 scales + f16 x + f16 y."""
    return n * k // 2 + n * (k // group) * 2 + m * k * 2 + m * n * 2


def gemm_flops(n: int, k: int, m: int) -> int:
    return 2 * m * n * k


def make_linear_cuda(n: int, k: int, group: int, seed: int, device, sigma: float = 0.02):
    """Same recipe as :func:`make_linear`, generated on the device with torch's seeded generator
    (used where a host round trip of tens of GB would dominate, e.g. the 64-layer stack).
    Returns (q int32 [n,k/8], s float16 [n,k/group]) CUDA tensors in the boundary format."""
    import torch
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    w = torch.randn((n, k // group, group), generator=gen, device=device, dtype=torch.float32) * sigma
    amax = w.abs().amax(dim=2)
    amax = torch.where(amax == 0, torch.full_like(amax, 1e-6), amax)
    s16 = (amax / 7.0).to(torch.float16)
    sf = s16.to(torch.float32)
    sf = torch.where(sf == 0, torch.full_like(sf, 2.0 ** -24), sf)
    nib = (torch.clamp(torch.round(w / sf[:, :, None]), -8, 7).to(torch.int32) + 8).reshape(n, k // 8, 8)
    del w
    shifts = (4 * torch.arange(8, device=device, dtype=torch.int64))[None, None, :]
    q = (nib.to(torch.int64) << shifts).sum(dim=2)
    q = torch.where(q >= 2 ** 31, q - 2 ** 32, q).to(torch.int32)
    return q.contiguous(), s16.contiguous()


def make_experts(n_exp: int, ffn: int, hidden: int, group: int, seed: int, sigma: float = 0.02):
    """Expert linears of one MoE layer, expert-major: w13 = gate rows then up rows [n_exp, 2*ffn, hidden],
    w2 = down [n_exp, hidden, ffn].  Returns (w13_q, w13_s, w2_q, w2_s) in the boundary format."""
    q13, s13 = make_linear(n_exp * 2 * ffn, hidden, group, seed, sigma)
    q2, s2 = make_linear(n_exp * hidden, ffn, group, seed + 1, sigma)
    return (q13.reshape(n_exp, 2 * ffn, hidden // 8), s13.reshape(n_exp, 2 * ffn, hidden // group),
            q2.reshape(n_exp, hidden, ffn // 8), s2.reshape(n_exp, hidden, ffn // group))
