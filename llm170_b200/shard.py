"""Tensor- and expert-parallel partitioning of W4A16 linears (host-side index arithmetic only).

The reference has no tensor parallelism (it rejects anything but 1 or 2 pipeline stages,
crates/server/src/main.rs:245-247); the partitioning below is what a rank uploads so that the library,
which has no collective of its own, computes its share:

* column-parallel (qkv, gate_up): rank r owns output rows [r*N/G, (r+1)*N/G); x is replicated; no collective.
  A fused gate|up matrix is split per half so that silu(gate)*up stays local.
* row-parallel (o_proj, down): rank r owns input channels [r*K/G, (r+1)*K/G) of every row -- whole scale
  groups -- and the partial outputs are summed over ranks (f16 all-reduce).
* experts: rank r owns experts [r*E/G, (r+1)*E/G).
"""
from __future__ import annotations

import numpy as np


def shard_linear(q: np.ndarray, s: np.ndarray, n: int, k: int, group: int, kind: str, rank: int, world: int,
                 fused_halves: int = 1):
    """(q u32 [n,k/8], s u16 [n,k/group]) -> this rank's (q, s, n', k')."""
    q = np.asarray(q).reshape(n, k // 8)
    s = np.asarray(s).reshape(n, k // group)
    if kind == "col":
        if n % (world * fused_halves * 16) != 0:
            raise ValueError(f"column-parallel: n={n} not divisible into {world}x{fused_halves} blocks of 16 rows")
        half = n // fused_halves
        per = half // world
        rows = np.concatenate([np.arange(h * half + rank * per, h * half + (rank + 1) * per) for h in range(fused_halves)])
        return np.ascontiguousarray(q[rows]), np.ascontiguousarray(s[rows]), rows.size, k
    if kind == "row":
        unit = max(group, 64)
        if k % (world * unit) != 0:
            raise ValueError(f"row-parallel: k={k} not divisible into {world} slices of whole {unit}-channel units")
        kp = k // world
        return (np.ascontiguousarray(q[:, rank * kp // 8:(rank + 1) * kp // 8]),
                np.ascontiguousarray(s[:, rank * kp // group:(rank + 1) * kp // group]), n, kp)
    raise ValueError(f"unknown parallel kind {kind!r}")


def shard_acts(x: np.ndarray, k: int, kind: str, rank: int, world: int) -> np.ndarray:
    """Activations a rank feeds its shard: replicated for column-parallel, the K slice for row-parallel."""
    x = np.asarray(x).reshape(-1, k)
    if kind == "col":
        return x
    kp = k // world
    return np.ascontiguousarray(x[:, rank * kp:(rank + 1) * kp])


def expert_range(n_experts: int, rank: int, world: int):
    if n_experts % world != 0:
        raise ValueError(f"{n_experts} experts do not split over {world} ranks")
    per = n_experts // world
    return rank * per, per
