"""Committed golden vectors (tests/golden/w4a16_golden.npz, made by tests/golden/make_golden.py):
the CPU oracle must reproduce them bit for bit, and the CUDA path must match them."""
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "w4a16_golden.npz")


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLD)


def test_oracle_reproduces_golden(orc, gold):
    for tag in ("g128", "g32"):
        n, k, g, t = gold[f"{tag}_shape"]
        q, s, x = gold[f"{tag}_q"], gold[f"{tag}_s"], gold[f"{tag}_x"]
        assert np.array_equal(orc.dequant_w4a16(q, s, n, k, g).view(np.uint32), gold[f"{tag}_deq"].view(np.uint32))
        assert np.array_equal(orc.linear_lane(q, s, x, t, n, k, g).view(np.uint32), gold[f"{tag}_y"].view(np.uint32))
    for i in range(4):
        sel = orc.select_topk(gold["topk_logits"][i], 4)
        assert [e for e, _ in sel] == gold["topk_idx"][i].tolist()
        assert np.array_equal(np.array([w for _, w in sel], np.float32), gold["topk_wt"][i])
    ne, kk, f, h, t = gold["moe_shape"]
    y = orc.moe_ffn(gold["moe_x"], gold["moe_logits"], gold["moe_w13_q"], gold["moe_w13_s"], gold["moe_w2_q"],
                    gold["moe_w2_s"], int(kk), 32)
    assert np.array_equal(y.view(np.uint32), gold["moe_y"].view(np.uint32))


def test_generator_is_reproducible(gold):
    from llm170_b200 import synth
    q, s = synth.make_linear(64, 256, 128, seed=1234)
    assert np.array_equal(q, gold["g128_q"]) and np.array_equal(s, gold["g128_s"])
    assert np.array_equal(synth.make_acts(3, 256, seed=4321), gold["g128_x"])


@pytest.mark.gpu
def test_cuda_path_matches_golden(gold):
    import torch
    from llm170_b200.w4a16_dec import W4a16Dec
    dec = W4a16Dec(0)
    try:
        for tag in ("g128", "g32"):
            n, k, g, t = (int(v) for v in gold[f"{tag}_shape"])
            dec.upload_lin_g("gold", gold[f"{tag}_q"], gold[f"{tag}_s"], n, k, g)
            assert np.array_equal(dec.dequant_lin("gold").cpu().numpy().view(np.uint32), gold[f"{tag}_deq"].view(np.uint32))
            x = torch.from_numpy(gold[f"{tag}_x"].view(np.float16).copy()).cuda()
            y = dec.lin_forward("gold", x, t).cpu().numpy()
            assert np.abs(y - gold[f"{tag}_y"]).max() <= 2e-3
            assert np.abs(y - gold[f"{tag}_y"]).max() <= 1e-5 * max(1.0, np.abs(gold[f"{tag}_y"]).max())
        ne, kk, f, h, t = (int(v) for v in gold["moe_shape"])
        dec.set_moe(ne, kk, f, h, 32)
        idx, wt = None, None
        dec.upload_experts(0, gold["moe_w13_q"], gold["moe_w13_s"], gold["moe_w2_q"], gold["moe_w2_s"])
        y = dec.moe_ffn_dev_t(0, torch.from_numpy(gold["moe_logits"]).cuda(),
                              torch.from_numpy(gold["moe_x"].view(np.float16).copy()).cuda(), t).cpu().numpy()
        assert np.abs(y - gold["moe_y"]).max() <= 2e-3
        dec.set_moe(16, 4, 64, 64, 32)
        idx, wt = dec.moe_topk(torch.from_numpy(gold["topk_logits"]).cuda())
        assert np.array_equal(idx.cpu().numpy(), gold["topk_idx"])
        assert np.allclose(wt.cpu().numpy(), gold["topk_wt"], rtol=0, atol=2e-7)
        dec.sync()
    finally:
        dec.close()
