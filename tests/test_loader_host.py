"""Host-side tests of the checkpoint reader (no GPU): the safetensors archive and the linear scan behind the C ABI,
and the directory-level checks of llm170_b200.w4a16_model, on the tiny checkpoints of tests/golden/tiny_w4a16
(written by tests/golden/make_tiny_st.py in the reference generator's format)."""
import json
import os
import struct

import numpy as np
import pytest

from llm170_b200.w4a16_dec import SafeTensors, W4a16Error
from llm170_b200.w4a16_model import check_quant

HERE = os.path.dirname(os.path.abspath(__file__))
TINY = os.path.join(HERE, "golden", "tiny_w4a16")


def read_st(path):
    """Independent numpy reader of one safetensors file: {name: (dtype, shape, bytes)}."""
    raw = open(path, "rb").read()
    hlen = struct.unpack("<Q", raw[:8])[0]
    hdr = json.loads(raw[8:8 + hlen])
    out = {}
    for name, e in hdr.items():
        if name != "__metadata__":
            a, b = e["data_offsets"]
            out[name] = (e["dtype"], e["shape"], raw[8 + hlen + a:8 + hlen + b])
    return out


def test_archive_lists_the_linears_and_skips_other_tensors():
    st = SafeTensors(os.path.join(TINY, "dense"))                      # a directory of model*.safetensors
    assert st.linears() == [("blk.0.attn_q", 64, 256, 128, False), ("blk.0.ffn_down", 48, 384, 128, False)]
    st2 = SafeTensors(os.path.join(TINY, "experts", "model.safetensors"))   # a single file
    assert st2.linears() == [("blk.0.ffn_down_exps.0", 64, 64, 32, True), ("blk.0.ffn_gate_exps.0", 32, 128, 32, True)]
    assert st.tag("blk.0.attn_q") != st.tag("blk.0.ffn_down")
    assert st.tag("blk.0.attn_q") == SafeTensors(os.path.join(TINY, "dense")).tag("blk.0.attn_q")
    with pytest.raises(W4a16Error):
        st.tag("nope")


def rewrite(tmp_path, mutate):
    """The dense checkpoint with its header passed through `mutate(header dict)`."""
    raw = open(os.path.join(TINY, "dense", "model.safetensors"), "rb").read()
    hlen = struct.unpack("<Q", raw[:8])[0]
    hdr = json.loads(raw[8:8 + hlen])
    mutate(hdr)
    hb = json.dumps(hdr).encode()
    p = tmp_path / "model.safetensors"
    p.write_bytes(struct.pack("<Q", len(hb)) + hb + raw[8 + hlen:])
    return str(p)


def test_archive_rejects_broken_headers_and_triples(tmp_path):
    # st.rs:213-290 and w4a16.rs:124-175: every contract violation is an error, never a crash
    def no_scale(h): del h["blk.0.attn_q.weight_scale"]
    def no_shape(h): del h["blk.0.attn_q.weight_shape"]
    def bad_dtype(h): h["blk.0.attn_q.weight_packed"]["dtype"] = "F16"
    def bad_bytes(h): h["blk.0.attn_q.weight_packed"]["data_offsets"][1] -= 4
    def reversed_offs(h): h["blk.0.attn_q.weight_packed"]["data_offsets"].reverse()
    def beyond(h):
        for e in h.values():
            if "data_offsets" in e:
                e["data_offsets"] = [e["data_offsets"][0] + 10 ** 9, e["data_offsets"][1] + 10 ** 9]
    def bad_group(h): h["blk.0.attn_q.weight_scale"]["shape"] = [64, 16]      # 256 / 16 = group 16
    def scale_f32(h): h["blk.0.attn_q.weight_scale"]["dtype"] = "F32"
    for m in (no_scale, no_shape, bad_dtype, bad_bytes, reversed_offs, beyond, bad_group, scale_f32):
        with pytest.raises(W4a16Error):
            SafeTensors(rewrite(tmp_path, m))
    with pytest.raises(W4a16Error):
        SafeTensors(str(tmp_path / "missing.safetensors"))
    (tmp_path / "short.safetensors").write_bytes(b"\x01\x02")
    with pytest.raises(W4a16Error):
        SafeTensors(str(tmp_path / "short.safetensors"))


def test_quant_config_rules():
    # w4a16.rs:193-236
    good = json.load(open(os.path.join(TINY, "experts", "quantization_config.json")))
    assert check_quant(good) == 32
    for mutate in (lambda c: c.update(quant_method="gptq"), lambda c: c.update(format="int-quantized") or
                   c["config_groups"]["group_0"].pop("format"),
                   lambda c: c["config_groups"]["group_0"]["weights"].update(num_bits=8),
                   lambda c: c["config_groups"]["group_0"]["weights"].update(symmetric=False),
                   lambda c: c["config_groups"]["group_0"]["weights"].update(group_size=16),
                   lambda c: c["config_groups"].update(group_1=c["config_groups"]["group_0"])):
        c = json.loads(json.dumps(good))
        mutate(c)
        with pytest.raises(W4a16Error):
            check_quant(c)


def test_fixture_matches_its_generator_recipe(orc):
    # the packed nibbles dequantise, with the stored scale, to within half a step of a weight the recipe can produce
    t = read_st(os.path.join(TINY, "experts", "model.safetensors"))
    q = np.frombuffer(t["blk.0.ffn_gate_exps.0.weight_packed"][2], "<u4").reshape(32, 16)
    s = np.frombuffer(t["blk.0.ffn_gate_exps.0.weight_scale"][2], "<u2").reshape(32, 4)
    assert struct.unpack("<qq", t["blk.0.ffn_gate_exps.0.weight_shape"][2]) == (32, 128)
    w = orc.dequant_w4a16(q, s, 32, 128, 32, scale_bf16=True)
    assert np.abs(w).max() < 0.05 * 2.0 + 1e-3 and np.abs(w).max() > 0.01
    nib = (q[:, :, None] >> (4 * np.arange(8, dtype=np.uint32))) & 0xF
    assert nib.max() == 15 or nib.min() == 1     # absmax / 7 scaling: every group reaches +-7
