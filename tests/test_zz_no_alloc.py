"""The allocation-free decode entry point (collected last on purpose).

``w4a16_sk_single_static`` serves hosts that cannot let a library call cudaMalloc -- an engine that owns the
whole device-memory budget, or a decode loop where an allocation's device-wide synchronisation is not
acceptable.  Its split-K scratch is a fixed array inside the library.  The test calls it through the C ABI
twice in a row and requires the same bits as the ordinary entry point, then checks that a launch whose
scratch would not fit is refused with a message instead of running.
"""
import numpy as np
import pytest
import torch

from llm170_b200 import synth

pytestmark = pytest.mark.gpu


def test_static_scratch_matches_regular_entry_twice():
    from llm170_b200.w4a16_dec import W4a16Dec, W4a16Error
    dec = W4a16Dec(0)
    try:
        for (n, k, group, t) in [(5120, 6144, 128, 1), (2048, 768, 32, 8), (7168, 5120, 128, 3)]:
            q, s = synth.make_linear(n, k, group, seed=n % 89 + t)
            dec.upload_lin_g("na", q, s, n, k, group)
            x = torch.from_numpy(synth.make_acts(t, k, seed=t).view(np.float16).copy()).cuda()
            ref = dec.sk_single_dev("na", x, t=t).clone()
            out = torch.empty_like(ref)
            for _ in range(2):                       # two calls in a row share the built-in array
                out.fill_(float("nan"))
                dec.sk_single_static("na", x, out=out, t=t)
                torch.cuda.synchronize()
                assert torch.equal(out, ref)         # same kernel, same split: bit-identical (tolerance 0)
            ref16 = dec.sk_single_dev("na", x, t=t, out_f16=True)
            assert torch.equal(dec.sk_single_static("na", x, t=t, out_f16=True), ref16)
        dec.kernel_status()
        # a launch that would need more than the built-in 8 MiB is refused, nothing runs: 8 tokens of a
        # 17408-channel input leave room for 31 units per CTA, so this 34816 x 17408 linear takes 597 CTAs
        # with two 8 KB parking slots each
        n, k = 34816, 17408
        q, s = synth.make_linear_cuda(n, k, 128, seed=1, device=torch.device("cuda", 0))
        dec.upload_lin_g_dev("big", q, s, n, k, 128)
        x = torch.randn((8, k), device="cuda").half()
        out = torch.full((8, n), 7.0, device="cuda")
        dec.set_tuning("gemv_persistent", 2)         # the persistent form at every token count
        try:
            with pytest.raises(W4a16Error, match="scratch"):
                dec.sk_single_static("big", x, out=out, t=8)
        finally:
            dec.set_tuning("gemv_persistent", 1)
        torch.cuda.synchronize()
        assert bool((out == 7.0).all())
        # one token fits (two CTAs per SM) and agrees
        assert torch.equal(dec.sk_single_static("big", x[:1], t=1), dec.sk_single_dev("big", x[:1], t=1))
        # the (row block, K split) form of the kernel has the same guard
        dec.set_tuning("gemv_persistent", 0)
        dec.set_tuning("gemv_ksplit", 16)            # 16 splits x 136 row blocks x 8 KB = 17 MB
        try:
            with pytest.raises(W4a16Error, match="scratch"):
                dec.sk_single_static("big", x[:1], out=out[:1], t=1)
            dec.set_tuning("gemv_ksplit", 0)
            assert torch.equal(dec.sk_single_static("big", x[:1], t=1), dec.sk_single_dev("big", x[:1], t=1))
        finally:
            dec.set_tuning("gemv_ksplit", 0)
            dec.set_tuning("gemv_persistent", 1)
    finally:
        dec.close()
