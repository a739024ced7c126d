"""Writes tests/golden/w4a16_golden.npz: small seeded inputs with the outputs of the KAT-pinned CPU oracle.

The reference is Rust and cannot run here, so these vectors come from the oracle restatement after it
passed the reference's known-answer tests (tests/test_oracle_kat.py).  They freeze its behaviour: a later
change to the oracle or to the synthetic generator that alters any bit fails tests/test_golden.py.
Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from llm170_b200 import synth  # noqa: E402


def build():
    out = {}
    for tag, (n, k, g, t) in {"g128": (64, 256, 128, 3), "g32": (32, 128, 32, 8)}.items():
        q, s = synth.make_linear(n, k, g, seed=1234)
        x = synth.make_acts(t, k, seed=4321)
        out[f"{tag}_q"], out[f"{tag}_s"], out[f"{tag}_x"] = q, s, x
        out[f"{tag}_deq"] = oracle.dequant_w4a16(q, s, n, k, g)
        out[f"{tag}_y"] = oracle.linear_lane(q, s, x, t, n, k, g, nthreads=1)
        out[f"{tag}_shape"] = np.array([n, k, g, t])
    lg = synth.make_router_logits(4, 16, seed=77)
    lg[0, 3] = lg[0, 9]  # a tie
    sel = [oracle.select_topk(lg[i], 4) for i in range(4)]
    out["topk_logits"] = lg
    out["topk_idx"] = np.array([[e for e, _ in r] for r in sel], np.int32)
    out["topk_wt"] = np.array([[w for _, w in r] for r in sel], np.float32)
    ne, kk, f, h, t = 4, 2, 64, 64, 6
    w = synth.make_experts(ne, f, h, 32, seed=55)
    xm = synth.make_acts(t, h, seed=56)
    lgm = synth.make_router_logits(t, ne, seed=57)
    out["moe_w13_q"], out["moe_w13_s"], out["moe_w2_q"], out["moe_w2_s"] = w
    out["moe_x"], out["moe_logits"] = xm, lgm
    out["moe_y"] = oracle.moe_ffn(xm, lgm, *w, kk, 32)
    out["moe_shape"] = np.array([ne, kk, f, h, t])
    return out


if __name__ == "__main__":
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "w4a16_golden.npz"), **build())
    print("written")
