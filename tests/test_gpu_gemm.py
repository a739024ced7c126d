"""GPU parity of the tensor-core prefill GEMM (t > 8) through the C ABI.

Three references:  (1) exact-arithmetic known-answer tests of the reference (bit equality);
(2) the value the kernel is specified to compute -- x times the dequantised weight rounded once
to f16, accumulated in f32 -- as a plain torch fp32 matmul (tolerance 1e-4 relative to the output
scale); (3) the f32-accumulated CPU lane oracle with the 2e-3 max-abs gate."""
import numpy as np
import pytest
import torch

from llm170_b200 import synth

pytestmark = pytest.mark.gpu
TOL = 2e-3


@pytest.fixture(scope="module")
def dec():
    from llm170_b200.w4a16_dec import W4a16Dec
    torch.backends.cuda.matmul.allow_tf32 = False
    d = W4a16Dec(0)
    yield d
    d.close()


def x_dev(x_u16):
    return torch.from_numpy(x_u16.view(np.float16).copy()).cuda()


def pow2_case(t, k, n, group):
    kk, nn = np.meshgrid(np.arange(k), np.arange(n))
    nib = ((kk * 7 + nn * 3) % 16).astype(np.uint32)
    q = np.bitwise_or.reduce(nib.reshape(n, k // 8, 8) << (4 * np.arange(8, dtype=np.uint32)), axis=2).astype(np.uint32)
    s = np.array([[(15 - ((r + g) % 5)) << 10 for g in range(k // group)] for r in range(n)], np.uint16)
    i = np.arange(t * k)
    x = ((15 - ((i // k + (i % k) // 8) % 4)) << 10).astype(np.uint16).reshape(t, k)
    w = (nib.astype(np.float64) - 8) * np.repeat(s.view(np.float16).astype(np.float64), group, axis=1)
    return q, s, x, (x.view(np.float16).astype(np.float64) @ w.T).astype(np.float32)


@pytest.mark.parametrize("t,k,n,group", [(16, 256, 128, 128), (64, 512, 256, 128), (300, 256, 272, 128),
                                         (33, 128, 64, 32), (129, 768, 512, 32)])
def test_pow2_kat_exact(dec, t, k, n, group):
    # crates/server/src/probes/w4a16/gpu/bench.rs:77-166: power-of-two scales/activations -> exact sums
    q, s, x, expect = pow2_case(t, k, n, group)
    dec.upload_lin_g("p2", q, s, n, k, group)
    y = dec.lin_forward("p2", x_dev(x), t)
    dec.sync()
    assert np.array_equal(y.cpu().numpy().view(np.uint32), expect.view(np.uint32))


@pytest.mark.parametrize("n,k,group,t", [(256, 128, 128, 9), (512, 1024, 128, 130), (1536, 2048, 32, 257),
                                         (2048, 768, 32, 64), (4096, 4096, 128, 16), (7168, 5120, 128, 512)])
def test_gemm_vs_f16_dequant_model_and_lane_oracle(dec, orc, n, k, group, t):
    q, s = synth.make_linear(n, k, group, seed=300 + t)
    x = synth.make_acts(t, k, seed=400 + t, scale=1.0 / np.sqrt(k))
    dec.upload_lin_g("g", q, s, n, k, group)
    xd = x_dev(x)
    y = dec.lin_forward("g", xd, t)
    dec.sync()
    w16 = dec.dequant_lin("g", f16=True)
    ref = xd.float() @ w16.float().T                       # plain torch fp32 reference of the specified op
    scale = ref.abs().max().item()
    assert (y - ref).abs().max().item() <= 1e-4 * scale + 1e-6
    rows = (0, min(n, 64))
    want = orc.linear_lane(q, s, x, t, n, k, group, rows=rows)
    got = y.cpu().numpy()[:, rows[0]:rows[1]]
    assert np.abs(got - want[:, rows[0]:rows[1]]).max() <= TOL
    y16 = dec.lin_forward("g", xd, t, out_f16=True)
    dec.sync()
    assert torch.equal(y16, y.to(torch.float16))
    dec.drop_lin("g")


@pytest.mark.parametrize("t,k,n,group", [(300, 256, 272, 128), (257, 768, 512, 32), (64, 512, 256, 128)])
def test_two_block_tiles_pow2_exact(dec, t, k, n, group):
    # the 256-token tile variant (two TMEM accumulators per CTA), forced, incl. ragged last tiles
    q, s, x, expect = pow2_case(t, k, n, group)
    dec.upload_lin_g("p2b", q, s, n, k, group)
    dec.set_tuning("gemm_mt", 2)
    try:
        y = dec.lin_forward("p2b", x_dev(x), t)
        dec.sync()
    finally:
        dec.set_tuning("gemm_mt", 0)
    assert np.array_equal(y.cpu().numpy().view(np.uint32), expect.view(np.uint32))


def test_tile_variants_agree_bitwise(dec):
    n, k, t = 1024, 2048, 700
    q, s = synth.make_linear(n, k, 128, seed=61)
    dec.upload_lin_g("mtv", q, s, n, k, 128)
    x = x_dev(synth.make_acts(t, k, seed=62, scale=1 / np.sqrt(k)))
    outs = []
    dec.set_tuning("gemm_ksplit", -1)         # one K range per tile: the tile variants then add in the same order
    for mt in (1, 2):
        dec.set_tuning("gemm_mt", mt)
        outs.append(dec.lin_forward("mtv", x, t).clone())
    dec.set_tuning("gemm_mt", 0)
    dec.set_tuning("gemm_ksplit", 0)
    dec.sync()
    assert torch.equal(outs[0], outs[1])      # same k order per output element -> same bits


@pytest.mark.parametrize("n,k,group,t,out_f16", [(512, 1024, 128, 512, 0), (1024, 2048, 128, 700, 0),
                                                  (784, 512, 32, 1300, 0), (2048, 2048, 32, 1024, 1),
                                                  (272, 128, 128, 130, 1), (256, 256, 128, 9, 1), (4864, 4096, 128, 512, 1)])
def test_tma_store_epilogue_agrees_bitwise_with_per_lane_stores(dec, n, k, group, t, out_f16):
    # the staged TMA-store epilogue writes the same values as the per-lane stores: ragged last token tile, a last
    # column chunk cut at n, both output types, and a launch whose last wave is split (those tiles keep their own path)
    q, s = synth.make_linear(n, k, group, seed=71 + t)
    dec.upload_lin_g("epi", q, s, n, k, group)
    x = x_dev(synth.make_acts(t, k, seed=72 + t, scale=1 / np.sqrt(k)))
    try:
        dec.set_tuning("gemm_tma_store", 0)
        lanes = dec.lin_forward("epi", x, t, out_f16=bool(out_f16)).clone()
        dec.set_tuning("gemm_tma_store", 1)
        guard = torch.full((t + 64, n), 7.0, device="cuda", dtype=torch.float16 if out_f16 else torch.float32)
        staged = dec.lin_forward("epi", x, t, dst=guard[:t], out_f16=bool(out_f16))
    finally:
        dec.set_tuning("gemm_tma_store", 1)
    dec.sync()
    assert torch.equal(lanes, staged)
    assert bool((guard[t:] == 7.0).all())        # nothing is written past the batch


def test_gemm_and_gemv_agree_on_the_same_weights(dec):
    # both kernels read the one resident copy; they differ only by the f16 rounding of the weight
    n, k = 1024, 2048
    q, s = synth.make_linear(n, k, 128, seed=12)
    dec.upload_lin_g("both", q, s, n, k, 128)
    x = x_dev(synth.make_acts(16, k, seed=13, scale=1 / np.sqrt(k)))
    y_gemm = dec.lin_forward("both", x, 16)
    y_gemv = torch.cat([dec.sk_single_dev("both", x[:8].contiguous(), t=8),
                        dec.sk_single_dev("both", x[8:].contiguous(), t=8)])
    dec.sync()
    assert (y_gemm - y_gemv).abs().max().item() <= 2e-4


# BASELINE config 3 at its own sizes: the four 27B-class layer shapes at M = 4096, and M = 1024 on the two largest.
# Every output is checked against the specified operation as a plain torch fp32 matmul (x times the weight rounded
# once to f16), and a spread of rows and tokens -- first, middle and last n-tile, first and last m-tile -- against
# the f32-accumulated CPU lane oracle with the 2e-3 gate (crates/server/src/probes/w4a16/gates.rs:108-138,
# crates/server/src/probes/w4a16/gpu/bench.rs:191-259 are the reference's checks of the same kernels).
@pytest.mark.parametrize("name,m", [("qkv", 4096), ("o_proj", 4096), ("gate_up", 4096), ("down", 4096),
                                    ("gate_up", 1024), ("down", 1024)])
def test_config3_prefill_shapes_full_size(dec, orc, name, m):
    k, n = synth.DENSE_27B[name]
    q, s = synth.make_linear_cuda(n, k, 128, seed=2000 + len(name), device=torch.device("cuda", 0))
    dec.upload_lin_g_dev("c3", q, s, n, k, 128)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(2)
    xd = (torch.randn((m, k), generator=gen, device="cuda") / (k ** 0.5)).to(torch.float16)
    y = dec.lin_forward("c3", xd, m)
    dec.sync()
    w16 = dec.dequant_lin("c3", f16=True)
    worst, scale = 0.0, 0.0
    for r0 in range(0, n, 8192):                      # row slabs keep the fp32 reference within a few GB
        ref = xd.float() @ w16[r0:r0 + 8192].float().T
        worst = max(worst, (y[:, r0:r0 + 8192] - ref).abs().max().item())
        scale = max(scale, ref.abs().max().item())
        del ref
    assert worst <= 1e-4 * scale + 1e-6, (worst, scale)
    # lane oracle on 3 x 32 rows and 64 tokens
    qh, sh = q.cpu().numpy().view(np.uint32), s.cpu().numpy().view(np.uint16)
    toks = np.r_[0:16, m // 2:m // 2 + 16, m - 32:m]
    xs = np.ascontiguousarray(xd[torch.from_numpy(toks).cuda()].cpu().numpy().view(np.uint16))
    got = y[torch.from_numpy(toks).cuda()].cpu().numpy()
    for r0 in (0, (n // 2) // 16 * 16, n - 32):
        want = orc.linear_lane(qh, sh, xs, len(toks), n, k, 128, rows=(r0, r0 + 32))
        assert np.abs(got[:, r0:r0 + 32] - want[:, r0:r0 + 32]).max() <= TOL
    y16 = dec.lin_forward("c3", xd, m, out_f16=True)
    dec.sync()
    assert torch.equal(y16, y.to(torch.float16))
    dec.drop_lin("c3")


# Split-K form of the GEMM (few tiles: the small-batch band above the decode GEMV, narrow linears): the partial
# tiles are added in split order by the last split to arrive, so forced splits reproduce the exact-arithmetic
# known answers bit for bit, twice in a row.
@pytest.mark.parametrize("t,k,n,group,ks", [(9, 1024, 128, 128, 4), (16, 2048, 272, 128, 8), (33, 1024, 512, 32, 3),
                                            (300, 1024, 272, 128, 2), (64, 4096, 256, 128, 16)])
def test_split_k_gemm_pow2_exact_and_repeatable(dec, t, k, n, group, ks):
    q, s, x, expect = pow2_case(t, k, n, group)
    dec.upload_lin_g("p2k", q, s, n, k, group)
    dec.set_tuning("gemm_ksplit", ks)
    try:
        y = dec.lin_forward("p2k", x_dev(x), t).clone()
        y2 = dec.lin_forward("p2k", x_dev(x), t)
        dec.sync()
        assert "split-K" in dec.last_kernel(), dec.last_kernel()
    finally:
        dec.set_tuning("gemm_ksplit", 0)
    assert np.array_equal(y.cpu().numpy().view(np.uint32), expect.view(np.uint32))
    assert torch.equal(y, y2)


# The small-batch band of the reference's FFMA family (crates/backend-gpu/src/rawcuda/assets/gptq4.cu:458-951,
# T <= 32, and the MTP verify width 9 of crates/backend-gpu/src/rawcuda/w4a16_dec/chains.rs:315-507) on the
# baseline's layer shapes: one call each, all tokens, rows spread over the output, against the lane oracle.
@pytest.mark.parametrize("name", ["qkv", "o_proj", "gate_up", "down"])
@pytest.mark.parametrize("t", [9, 16, 32])
def test_small_batch_band_on_layer_shapes(dec, orc, name, t):
    k, n = synth.DENSE_27B[name]
    q, s = synth.make_linear_cuda(n, k, 128, seed=77, device=torch.device("cuda", 0))
    dec.upload_lin_g_dev("sb", q, s, n, k, 128)
    x = synth.make_acts(t, k, seed=t)
    y = dec.lin_forward("sb", x_dev(x), t)
    dec.sync()
    qh, sh = q.cpu().numpy().view(np.uint32), s.cpu().numpy().view(np.uint16)
    got = y.cpu().numpy()
    scale = 0.0
    for r0 in (0, (n // 2) // 16 * 16, n - 64):
        want = orc.linear_lane(qh, sh, x, t, n, k, 128, rows=(r0, r0 + 64))
        scale = max(scale, float(np.abs(want).max()))
        # N(0,1) activations: |y| reaches ~10, and the GEMM multiplies weights rounded once to f16 (relative 2^-11)
        assert np.abs(got[:, r0:r0 + 64] - want[:, r0:r0 + 64]).max() <= TOL * max(1.0, scale)
    dec.drop_lin("sb")


def test_last_wave_split_agrees_with_whole_tiles(dec):
    # 19 x 8 = 152 tiles of 256 tokens on 148 SMs: the automatic choice runs 148 whole tiles and splits the last 4 along K;
    # same products, partial sums added in another order -> agreement to f32 rounding, and bit-repeatable
    n, k, t = 2048, 4096, 4864
    q, s = synth.make_linear_cuda(n, k, 128, seed=5, device=torch.device("cuda", 0))
    dec.upload_lin_g_dev("lw", q, s, n, k, 128)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(9)
    x = (torch.randn((t, k), generator=gen, device="cuda") / (k ** 0.5)).to(torch.float16)
    y = dec.lin_forward("lw", x, t).clone()
    name = dec.last_kernel()
    y2 = dec.lin_forward("lw", x, t).clone()
    dec.set_tuning("gemm_ksplit", -1)
    try:
        y_whole = dec.lin_forward("lw", x, t)
        dec.sync()
    finally:
        dec.set_tuning("gemm_ksplit", 0)
    if torch.cuda.get_device_properties(0).multi_processor_count == 148:
        assert "last wave" in name, name
    assert torch.equal(y, y2)
    assert (y - y_whole).abs().max().item() <= 1e-5 * y_whole.abs().max().item() + 1e-7
    dec.drop_lin("lw")
