"""Mirror of the reference's ``W4a16Model`` (crates/core/src/w4a16.rs:100-245): a compressed-tensors
``pack-quantized`` checkpoint directory -- its quantisation config checked, its linears listed -- plus what the
reference does not have: a cache of the device tile layout, so that a second load is plain copies.

The archive reader and the uploads run behind the C ABI (``w4a16_st_*``, ``w4a16_upload_lin_st``,
``w4a16_save_lin_cache`` / ``w4a16_load_lin_cache``); this file holds the directory-level policy only.
"""
from __future__ import annotations

import json
import os

from .w4a16_dec import SafeTensors, W4a16Dec, W4a16Error


def check_quant(cfg: dict) -> int:
    """w4a16.rs:193-236: compressed-tensors, pack-quantized, int4 symmetric, one scheme, group 32/64/128.
    Returns the group size of the config."""
    if cfg.get("quant_method", "") != "compressed-tensors":
        raise W4a16Error(f"quant_method={cfg.get('quant_method')!r}")
    groups = cfg.get("config_groups")
    if not isinstance(groups, dict):
        raise W4a16Error("config_groups missing")
    if len(groups) != 1:
        raise W4a16Error(f"config_groups has {len(groups)} schemes; a single scheme is supported")
    g0 = next(iter(groups.values()))
    fmt = g0.get("format") or cfg.get("format") or ""
    if fmt != "pack-quantized":
        raise W4a16Error(f"format={fmt!r}")
    w = g0.get("weights")
    if not isinstance(w, dict):
        raise W4a16Error("group weights missing")
    bits, group, sym = int(w.get("num_bits", 0)), int(w.get("group_size", 0)), bool(w.get("symmetric", False))
    if bits != 4 or not sym:
        raise W4a16Error(f"bits={bits} sym={sym}: int4 symmetric only")
    if group not in (32, 64, 128):
        raise W4a16Error(f"group={group}: only 32, 64, 128")
    return group


def _find_key(node, key):
    """First value stored under `key` anywhere in a JSON tree (the reference scans config.json for the key wherever
    it is nested, e.g. under text_config: w4a16.rs:493-535)."""
    if isinstance(node, dict):
        if key in node:
            return node[key]
        for v in node.values():
            r = _find_key(v, key)
            if r is not None:
                return r
    elif isinstance(node, list):
        for v in node:
            r = _find_key(v, key)
            if r is not None:
                return r
    return None


class W4a16Model:
    def __init__(self, directory: str):
        """W4a16Model::open (w4a16.rs:107-191)."""
        self.dir = directory
        cfg = None
        for f in ("quantization_config.json", "quant_config.json"):
            p = os.path.join(directory, f)
            if os.path.exists(p):
                cfg = json.load(open(p))
                break
        if cfg is None:
            p = os.path.join(directory, "config.json")
            if not os.path.exists(p):
                raise W4a16Error("config.json missing")
            cfg = _find_key(json.load(open(p)), "quantization_config")
            if not isinstance(cfg, dict):
                raise W4a16Error("config.json holds no quantization_config")
        self.group = check_quant(cfg)
        self.st = SafeTensors(directory)
        self.lins = {base: (n, k, g, bf) for base, n, k, g, bf in self.st.linears()}
        if not self.lins:
            raise W4a16Error("no weight_packed tensor: not a W4A16 checkpoint")

    def close(self):
        self.st.close()

    def scale_is_bf16(self, base: str) -> bool:
        return self.lins[base][3]

    def upload_all(self, dec: W4a16Dec, cache_dir: str | None = None):
        """Every linear under its tensor name.  With `cache_dir`, a linear whose cache file matches its source tag is
        read back from it (plain copies); the others are re-tiled from the checkpoint and their cache file written.
        Returns {base: "cache" | "checkpoint"}."""
        how = {}
        if cache_dir:
            os.makedirs(cache_dir, exist_ok=True)
        for base in sorted(self.lins):
            tag = self.st.tag(base)
            path = os.path.join(cache_dir, base.replace("/", "_") + ".w4t64") if cache_dir else None
            if path and os.path.exists(path):
                try:
                    dec.load_lin_cache(base, path, tag)
                    how[base] = "cache"
                    continue
                except W4a16Error:
                    pass   # stale or foreign file: rebuild it below
            dec.upload_lin_st(base, self.st, base)
            if path:
                dec.save_lin_cache(base, path, tag)
            how[base] = "checkpoint"
        return how
