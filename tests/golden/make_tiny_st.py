#!/usr/bin/env python3
"""Writes the two tiny compressed-tensors checkpoints under tests/golden/tiny_w4a16/ that the loader tests read.

File format and quantiser recipe are those of the reference's fixture generator (scripts/gen_tiny_w4a16.py:4-66):
a 64-bit LCG, each weight the sum of four uniforms in [-0.5, 0.5) times sigma, one scale = absmax / 7 per group --
stored as F16 for group 128 and as BF16 (the upper half of the f32) for group 32 --
q = clamp(round(w / scale), -8, 7), nibble q+8 at bits 4*(i&7) of little-endian word i>>3; per linear the tensors
`<base>.weight_packed` I32 [n, k/8], `<base>.weight_scale` [n, k/group], `<base>.weight_shape` I64 [2];
a safetensors file = u64 header length, JSON header {name: {dtype, shape, data_offsets}}, data.  Sizes are smaller.
Run from the repository root:  python tests/golden/make_tiny_st.py
"""
import json
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
MASK = (1 << 64) - 1


class Lcg:
    def __init__(self, seed):
        self.x = seed & MASK

    def uniforms(self, count):
        out = np.empty(count, np.float64)
        x = self.x
        for i in range(count):
            x = (x * 6364136223846793005 + 1442695040888963407) & MASK
            out[i] = (x >> 11) / float(1 << 53) - 0.5
        self.x = x
        return out


def quantised_triple(rng, n, k, group, sigma=0.05):
    """(packed u32 [n,k/8], scale bits u16 [n,k/group], dtype name) of one linear."""
    w = rng.uniforms(n * k * 4).reshape(n, k, 4).sum(axis=2) * sigma
    wg = w.reshape(n, k // group, group)
    amax = np.abs(wg).max(axis=2)
    s = np.where(amax == 0, 1e-6, amax) / 7.0
    q = np.clip(np.rint(wg / s[:, :, None]), -8, 7).astype(np.int64) + 8
    nib = q.reshape(n, k // 8, 8).astype(np.uint32)
    packed = np.bitwise_or.reduce(nib << (4 * np.arange(8, dtype=np.uint32)), axis=2).astype("<u4")
    if group == 128:
        return packed, s.astype("<f2").view("<u2"), "F16"
    return packed, (s.astype("<f4").view("<u4") >> 16).astype("<u2"), "BF16"


def write_safetensors(path, tensors):
    """tensors: {name: (dtype name, shape, bytes)}; entries are laid out in name order."""
    header, blob = {"__metadata__": {"format": "pt"}}, bytearray()
    for name in sorted(tensors):
        dtype, shape, data = tensors[name]
        header[name] = {"dtype": dtype, "shape": list(shape), "data_offsets": [len(blob), len(blob) + len(data)]}
        blob += data
    hb = json.dumps(header).encode()
    os.makedirs(os.path.dirname(path), exist_ok=True)
    with open(path, "wb") as f:
        f.write(np.uint64(len(hb)).astype("<u8").tobytes())
        f.write(hb)
        f.write(blob)


def add_linear(tensors, rng, base, n, k, group):
    packed, scale, sdt = quantised_triple(rng, n, k, group)
    tensors[base + ".weight_packed"] = ("I32", packed.shape, packed.tobytes())
    tensors[base + ".weight_scale"] = (sdt, scale.shape, scale.tobytes())
    tensors[base + ".weight_shape"] = ("I64", (2,), np.array([n, k], "<i8").tobytes())


def quant_cfg(group):
    return {"quant_method": "compressed-tensors", "format": "pack-quantized",
            "config_groups": {"group_0": {"format": "pack-quantized",
                                          "weights": {"num_bits": 4, "symmetric": True, "group_size": group}}}}


def main():
    root = os.path.join(HERE, "tiny_w4a16")
    # dense: group 128, F16 scales, beside a non-quantised tensor the scan must skip
    rng, t = Lcg(0xC0FFEE), {}
    add_linear(t, rng, "blk.0.attn_q", 64, 256, 128)
    add_linear(t, rng, "blk.0.ffn_down", 48, 384, 128)
    norm = (rng.uniforms(256).astype("<f4").view("<u4") >> 16).astype("<u2")
    t["blk.0.attn_norm.weight"] = ("BF16", (256,), norm.tobytes())
    write_safetensors(os.path.join(root, "dense", "model.safetensors"), t)
    with open(os.path.join(root, "dense", "config.json"), "w") as f:
        json.dump({"architectures": ["tiny"], "quantization_config": quant_cfg(128)}, f)
    # experts: group 32, BF16 scales
    rng, t = Lcg(0xBEEF), {}
    add_linear(t, rng, "blk.0.ffn_gate_exps.0", 32, 128, 32)
    add_linear(t, rng, "blk.0.ffn_down_exps.0", 64, 64, 32)
    write_safetensors(os.path.join(root, "experts", "model.safetensors"), t)
    with open(os.path.join(root, "experts", "quantization_config.json"), "w") as f:
        json.dump(quant_cfg(32), f)
    print("written", root)


if __name__ == "__main__":
    main()
