"""GPU parity of the resident layout, the dequantiser and the decode GEMV against the CPU oracle.
All calls go through the C ABI (llm170_b200.W4a16Dec / Gptq4 are thin ctypes wrappers)."""
import numpy as np
import pytest
import torch

from llm170_b200 import synth

pytestmark = pytest.mark.gpu

TOL = 2e-3  # max-abs gate on the f32 output against the f32-accumulated lane oracle


@pytest.fixture(scope="module")
def dec():
    from llm170_b200.w4a16_dec import W4a16Dec
    d = W4a16Dec(0)
    yield d
    d.close()


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def x_dev(x_u16):
    return torch.from_numpy(x_u16.view(np.float16).copy()).cuda()


@pytest.mark.parametrize("n,k,group", [(128, 256, 128), (64, 64, 32), (272, 1216, 32), (4096, 4096, 128)])
def test_repack_roundtrip_and_dequant_bit_exact(dec, orc, n, k, group):
    q, s = synth.make_linear(n, k, group, seed=n + k)
    dec.upload_lin_g("t", q, s, n, k, group)
    assert dec.lin_spec("t") == (n, k, group)
    q2, s2 = dec.unpack_lin("t")
    assert np.array_equal(q2.cpu().numpy().view(np.uint32), q)
    assert np.array_equal(s2.cpu().numpy().view(np.uint16), s)
    want = orc.dequant_w4a16(q, s, n, k, group)
    got = dec.dequant_lin("t").cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))           # D1: bit-exact vs lane/cpu.rs
    got16 = dec.dequant_lin("t", f16=True).cpu().numpy()
    assert np.array_equal(got16.view(np.uint16), want.astype(np.float16).view(np.uint16))  # D2 = RN_f16(D1)


def test_repack_kat_lcg_roundtrip(dec):
    # same generator as the reference's round-trip test (crates/core/src/marlin.rs:107-122)
    n, k = 128, 64
    seed, M64 = 0x123456789ABCDEF0, (1 << 64) - 1
    q = np.zeros(n * (k // 8), np.uint32)
    for i in range(q.size):
        seed = (seed * 6364136223846793005 + 1442695040888963407) & M64
        q[i] = seed >> 32
    dec.upload_lin_g("kat", q.reshape(n, k // 8), np.full((n, 2), 0x3C00, np.uint16), n, k, 32)
    q2, _ = dec.unpack_lin("kat")
    assert np.array_equal(q2.cpu().numpy().view(np.uint32).ravel(), q)


def test_upload_contract_errors(dec):
    from llm170_b200.w4a16_dec import W4a16Error
    q, s = synth.make_linear(64, 128, 128, seed=1)
    with pytest.raises(W4a16Error):      # length mismatch (upload.rs:27-33)
        dec.upload_lin_g("bad", q[:-1], s, 64, 128, 128)
    with pytest.raises(W4a16Error):      # unsupported group (gptq4.rs:60-70)
        dec.upload_lin_g("bad", q, s, 64, 128, 64)
    with pytest.raises(W4a16Error):      # n not a multiple of the tile
        dec.upload_lin_g("bad", q[:8], s[:8], 8, 128, 128)
    with pytest.raises(W4a16Error):
        dec.lin_spec("bad")
    with pytest.raises(W4a16Error):
        dec.sk_single_dev("nope", torch.zeros(128, dtype=torch.float16, device="cuda"))


def test_upload_replaces_by_name_and_counts_bytes(dec):
    base = dec.weights_bytes()
    q, s = synth.make_linear(64, 128, 128, seed=2)
    dec.upload_lin_g("rep", q, s, 64, 128, 128)
    assert dec.weights_bytes() == base + q.nbytes + s.nbytes
    q2, s2 = synth.make_linear(128, 256, 128, seed=3)
    dec.upload_lin_g("rep", q2, s2, 128, 256, 128)
    assert dec.lin_spec("rep") == (128, 256, 128)
    assert dec.weights_bytes() == base + q2.nbytes + s2.nbytes
    dec.drop_lin("rep")
    assert dec.weights_bytes() == base


def test_bf16_scales_exact_or_rejected(dec, orc):
    from llm170_b200.w4a16_dec import W4a16Error
    n, k = 64, 128
    q, _ = synth.make_linear(n, k, 32, seed=5)
    s_bf = np.array([[(127 - ((r + g) % 5)) << 7 for g in range(k // 32)] for r in range(n)], np.uint16)
    dec.upload_lin_g("bf", q, s_bf, n, k, 32, True)
    want = orc.dequant_w4a16(q, s_bf, n, k, 32, scale_bf16=True)
    assert np.array_equal(dec.dequant_lin("bf").cpu().numpy(), want)
    s_bad = s_bf.copy()
    s_bad[0, 0] = 0x0080  # 2^-126: not an f16 value
    with pytest.raises(W4a16Error):
        dec.upload_lin_g("bf2", q, s_bad, n, k, 32, True)


@pytest.mark.parametrize("subn", [1, 0])
@pytest.mark.parametrize("ksplit", [1, 2, 4, -1])
def test_decode_selfcheck_kat(dec, ksplit, subn):
    # crates/backend-gpu/src/rawcuda/w4a16_dec/probe.rs:1291-1426: scale = x = 1 -> y = sum(nib-8), bit-exact,
    # for split-K 1/2/4 and for a two-segment launch.
    n, k = 256, 512
    i = np.arange(n * k // 8, dtype=np.uint64)
    q = (((i * 0x9E3779B9) & 0xFFFFFFFF) ^ 0x12345678).astype(np.uint32).reshape(n, k // 8)
    s = np.full((n, k // 128), 0x3C00, np.uint16)
    nib = ((q[:, :, None] >> (4 * np.arange(8, dtype=np.uint32))) & 0xF).astype(np.int64) - 8
    want = nib.reshape(n, -1).sum(axis=1).astype(np.float32)
    dec.upload_lin_g("sc", q, s, n, k, 128)
    x = torch.ones(k, dtype=torch.float16, device="cuda")
    # ksplit >= 1: the (row block, K split) form of the kernel; -1: the persistent form
    dec.set_tuning("gemv_persistent", 2 if ksplit < 0 else 0)
    dec.set_tuning("gemv_ksplit", max(ksplit, 0))
    dec.set_tuning("gemv_subnormal", subn)
    try:
        y = dec.sk_single_dev("sc", x).cpu().numpy()[0]
        assert np.array_equal(y.view(np.uint32), want.view(np.uint32))
        y1, y2 = dec.sk_multi_dev(["sc", "sc"], x)
        assert np.array_equal(y1.cpu().numpy()[0], want) and np.array_equal(y2.cpu().numpy()[0], want)
    finally:
        dec.set_tuning("gemv_ksplit", 0)
        dec.set_tuning("gemv_subnormal", 1)
        dec.set_tuning("gemv_persistent", 1)


@pytest.mark.parametrize("subn", [1, 0])
@pytest.mark.parametrize("t", [1, 3, 8])
def test_pow2_kat_exact(dec, orc, t, subn):
    # crates/server/src/probes/w4a16/gpu/bench.rs:77-121: power-of-two scales and activations make
    # every partial sum exact, so the GPU result must equal the f64 expectation bit for bit.
    k, n = 256, 128
    kk, nn = np.meshgrid(np.arange(k), np.arange(n))
    nib = ((kk * 7 + nn * 3) % 16).astype(np.uint32)
    q = np.bitwise_or.reduce(nib.reshape(n, k // 8, 8) << (4 * np.arange(8, dtype=np.uint32)), axis=2).astype(np.uint32)
    s = np.array([[(15 - ((r + g) % 5)) << 10 for g in range(k // 128)] for r in range(n)], np.uint16)
    i = np.arange(t * k)
    x = ((15 - ((i // k + (i % k) // 8) % 4)) << 10).astype(np.uint16).reshape(t, k)
    expect = (x.view(np.float16).astype(np.float64) @
              ((nib.astype(np.float64) - 8) * np.repeat(s.view(np.float16).astype(np.float64), 128, axis=1)).T
              ).astype(np.float32)
    dec.upload_lin_g("p2", q, s, n, k, 128)
    dec.set_tuning("gemv_subnormal", subn)
    try:
        y = dec.lin_forward("p2", x_dev(x), t).cpu().numpy()
    finally:
        dec.set_tuning("gemv_subnormal", 1)
    assert np.array_equal(y.view(np.uint32), expect.view(np.uint32))


@pytest.mark.parametrize("n,k,group,t", [
    (4096, 4096, 128, 1), (4096, 4096, 128, 8), (1024, 5120, 128, 2), (1536, 2048, 32, 4),
    (2048, 768, 32, 1), (2048, 768, 32, 8), (48, 192, 32, 5), (16, 128, 128, 7), (5120, 17408, 128, 1),
    (5120, 17408, 128, 8),
])
def test_gemv_vs_lane_oracle(dec, orc, n, k, group, t):
    q, s = synth.make_linear(n, k, group, seed=100 + n % 97 + t)
    x = synth.make_acts(t, k, seed=200 + t)
    dec.upload_lin_g("g", q, s, n, k, group)
    rows = (0, n) if n * k * t <= (1 << 28) else (n // 2 - 256, n // 2 + 256)
    want = orc.linear_lane(q, s, x, t, n, k, group, rows=rows)
    try:
        for form in (2, 0):                  # the persistent form, then the (row block, K split) form
            dec.set_tuning("gemv_persistent", form)
            y = dec.lin_forward("g", x_dev(x), t)
            got = y.cpu().numpy()[:, rows[0]:rows[1]]
            err = np.abs(got.astype(np.float64) - want[:, rows[0]:rows[1]]).max()
            assert err <= TOL, (form, err)
            # f16 output is the f32 result rounded once
            y16 = dec.lin_forward("g", x_dev(x), t, out_f16=True).cpu().numpy()
            assert np.array_equal(y16.view(np.uint16), y.cpu().numpy().astype(np.float16).view(np.uint16))
    finally:
        dec.set_tuning("gemv_persistent", 1)
    dec.drop_lin("g")


def test_both_operand_forms_agree(dec, orc):
    # raw-nibble subnormal operands + per-group fix-up vs exact (nibble-8) operands: same sums up to f32 rounding
    n, k, t = 1024, 5120, 8
    q, s = synth.make_linear(n, k, 128, seed=21)
    x = x_dev(synth.make_acts(t, k, seed=22))
    dec.upload_lin_g("ab", q, s, n, k, 128)
    a = dec.sk_single_dev("ab", x, t=t).clone()
    dec.set_tuning("gemv_subnormal", 0)
    try:
        b = dec.sk_single_dev("ab", x, t=t).clone()
    finally:
        dec.set_tuning("gemv_subnormal", 1)
    assert (a - b).abs().max().item() <= 5e-5
    dec.kernel_status()


def test_config1_reference_cpu_case(dec, orc):
    # BASELINE config 1 (M=16 is served by the GEMM path; here the GEMV covers it as two calls of 8)
    n = k = 4096
    q, s = synth.make_linear(n, k, 128, seed=0)
    x = synth.make_acts(16, k, seed=0)
    want = orc.linear_lane(q, s, x, 16, n, k, 128)
    dec.upload_lin_g("c1", q, s, n, k, 128)
    xd = x_dev(x)
    got = torch.cat([dec.sk_single_dev("c1", xd[:8].contiguous(), t=8), dec.sk_single_dev("c1", xd[8:].contiguous(), t=8)])
    assert np.abs(got.cpu().numpy() - want).max() <= TOL
    dec.drop_lin("c1")


def test_config1_single_call_all_rows(dec, orc):
    # BASELINE config 1 through ONE lin_forward(t=16) call (the small-batch band above the decode GEMV),
    # every one of the 16 x 4096 outputs against the lane oracle; f16 output = RN_f16 of the f32 one
    n = k = 4096
    q, s = synth.make_linear(n, k, 128, seed=0)
    x = synth.make_acts(16, k, seed=0)
    want = orc.linear_lane(q, s, x, 16, n, k, 128)
    dec.upload_lin_g("c1b", q, s, n, k, 128)
    xd = x_dev(x)
    got = dec.lin_forward("c1b", xd, 16)
    dec.sync()
    assert np.abs(got.cpu().numpy() - want).max() <= TOL
    got16 = dec.lin_forward("c1b", xd, 16, out_f16=True)
    dec.sync()
    assert torch.equal(got16, got.to(torch.float16))
    dec.drop_lin("c1b")


def test_multi_segment_matches_single(dec):
    k = 1024
    segs = [("q_", 512), ("k_", 128), ("v_", 144)]
    x = x_dev(synth.make_acts(4, k, seed=9))
    for i, (nm, n) in enumerate(segs):
        q, s = synth.make_linear(n, k, 128, seed=40 + i)
        dec.upload_lin_g(nm, q, s, n, k, 128)
    outs = dec.sk_multi_dev([nm for nm, _ in segs], x, t=4)
    outs2 = dec.sk_multi_dev([nm for nm, _ in segs], x, t=4)
    for (nm, _), o, o2 in zip(segs, outs, outs2):
        assert torch.equal(o, o2)                      # the same launch twice: the same bits
        # the leftover row blocks of a launch are cut along K by the launch's geometry, so the multi-segment
        # launch and the single one may add the same f32 terms in another order
        single = dec.sk_single_dev(nm, x, t=4)
        assert (o - single).abs().max().item() <= 1e-5 * max(1.0, single.abs().max().item())


def test_split_k_is_deterministic_and_scratch_is_clean(dec):
    n, k = 512, 4096
    q, s = synth.make_linear(n, k, 128, seed=77)
    dec.upload_lin_g("det", q, s, n, k, 128)
    x = x_dev(synth.make_acts(8, k, seed=78))
    ref = dec.sk_single_dev("det", x, t=8).clone()
    for ks in (2, 8, 16):
        dec.set_tuning("gemv_ksplit", ks)
        a = dec.sk_single_dev("det", x, t=8).clone()
        b = dec.sk_single_dev("det", x, t=8).clone()
        assert torch.equal(a, b)                      # same split -> same bits, tickets were reset
        assert (a - ref).abs().max().item() < 1e-3
    dec.set_tuning("gemv_ksplit", 0)


def test_graph_capture_replay(dec):
    n, k = 1024, 2048
    q, s = synth.make_linear(n, k, 128, seed=31)
    dec.upload_lin_g("gr", q, s, n, k, 128)
    x = x_dev(synth.make_acts(1, k, seed=32))
    eager = dec.sk_single_dev("gr", x).clone()         # also warms scratch
    out = torch.zeros_like(eager)
    torch.cuda.synchronize()
    st = torch.cuda.ExternalStream(dec.stream_ptr())
    with torch.cuda.stream(st):
        dec.capture_begin()
        dec.sk_single_dev("gr", x, out=out)
        g = dec.capture_end()
    for _ in range(3):
        out.zero_()
        torch.cuda.synchronize()
        dec.graph_launch(g)
        dec.sync()
        assert torch.equal(out, eager)
    dec.graph_destroy(g)


def test_host_buffer_forward_and_gptq4_gate(dec, orc):
    # crates/server/src/probes/w4a16/gates.rs:108-138: rows<=4 of a linear, x uniform [-1,1) -> f16,
    # GPU f32 output against dot_row_w4a16_lane_group; the reference accepts <=1e-5 at t=1.
    from llm170_b200.gptq4 import Gptq4
    n, k, group = 64, 5120, 128
    q, s = synth.make_linear(n, k, group, seed=55)
    rng = np.random.default_rng(5)
    x = (rng.random((8, k), dtype=np.float32) * 2 - 1).astype(np.float16).view(np.uint16)
    want = orc.linear_lane(q, s, x, 8, n, k, group)
    g4 = Gptq4.__new__(Gptq4)
    g4.dec = dec
    got8 = g4.gemm(x, 8, q, s, n, k, group)
    got1 = g4.gemv(x[0], q, s, n, k, group)
    assert np.abs(got8 - want).max() <= 1e-4
    assert np.abs(got1[0] - want[0]).max() <= 1e-4
    dec.upload_lin_g("hb", q, s, n, k, group)
    y = dec.lin_forward_host("hb", x, 8)
    assert np.array_equal(y, got8)


@pytest.mark.parametrize("rowblock", [0, 1])
def test_debug_timeline_stamps_are_ordered(dec, rowblock):
    # w4a16_debug_timeline: every CTA of a decode launch stamps entry <= dependency wait <= x staged <= main loop
    # start <= main loop end <= exit (nanoseconds of the global timer), then its SM id and unit count; kept by the
    # persistent form (gemv_rowblock = 0) and by the row-block form alike
    n, k = 2048, 1024
    q, s = synth.make_linear(n, k, 128, seed=3)
    dec.upload_lin_g("tl", q, s, n, k, 128)
    x = x_dev(synth.make_acts(1, k, seed=4))
    dec.set_tuning("gemv_rowblock", rowblock)
    ref = dec.sk_single_dev("tl", x).clone()
    assert dec.last_kernel().startswith("gemv_ru_kernel" if rowblock else "gemv_sk_kernel")
    dec.set_tuning("debug_timeline", 1)
    try:
        c0 = dec.launch_count()
        y = dec.sk_single_dev("tl", x)
        tl = dec.debug_timeline().reshape(64, 384, 16)[c0 % 64]
        live = tl[tl[:, 0] > 0]
        assert len(live) > 0 and len(live) <= 384
        for a, b in ((0, 1), (1, 2), (2, 3), (3, 4), (4, 5)):
            assert (live[:, a] <= live[:, b]).all(), (a, b)
        assert (live[:, 7] >= 1).all() and (live[:, 6] >= 0).all() and (live[:, 6] < 256).all()
        assert torch.equal(y, ref)            # the stamps do not change the result
    finally:
        dec.set_tuning("debug_timeline", 0)
        dec.set_tuning("gemv_rowblock", 1)
    with pytest.raises(Exception):
        dec.debug_timeline()                  # off again: the call says so


def test_captured_graph_survives_scratch_growth(dec):
    # a graph captured with a small shape keeps the scratch addresses of that time; a later eager call that needs
    # more scratch must not free them under the graph
    n, k = 512, 2048
    q, s = synth.make_linear(n, k, 128, seed=5)
    dec.upload_lin_g("gsmall", q, s, n, k, 128)
    x = x_dev(synth.make_acts(1, k, seed=5))
    ref = dec.sk_single_dev("gsmall", x, t=1).clone()
    out = torch.zeros_like(ref)
    st = torch.cuda.ExternalStream(dec.stream_ptr(), device=torch.device("cuda", 0))
    torch.cuda.synchronize()
    with torch.cuda.stream(st):
        dec.capture_begin()
        dec.sk_single_dev("gsmall", x, out=out, t=1)
        gx = dec.capture_end()
    dec.graph_launch(gx)
    dec.sync()
    assert torch.equal(out, ref)
    # grow: forced K splits of a wide linear need far more partial-sum scratch than anything above
    nb, kb = 34816, 5120
    qb, sb = synth.make_linear_cuda(nb, kb, 128, seed=6, device=torch.device("cuda", 0))
    dec.upload_lin_g_dev("gbig", qb, sb, nb, kb, 128)
    dec.set_tuning("gemv_persistent", 0)
    dec.set_tuning("gemv_cluster", 0)
    dec.set_tuning("gemv_ksplit", 40)
    try:
        dec.sk_single_dev("gbig", torch.randn((8, kb), device="cuda").half(), t=8)
        dec.sync()
    finally:
        dec.set_tuning("gemv_ksplit", 0)
        dec.set_tuning("gemv_cluster", 1)
        dec.set_tuning("gemv_persistent", 1)
    out.zero_()
    dec.graph_launch(gx)
    dec.sync()
    assert torch.equal(out, ref)
    dec.graph_destroy(gx)
    dec.drop_lin("gbig")


def test_misaligned_buffers_are_refused_before_launch(dec):
    from llm170_b200.w4a16_dec import W4a16Error
    n, k = 256, 512
    q, s = synth.make_linear(n, k, 128, seed=8)
    dec.upload_lin_g("al", q, s, n, k, 128)
    x = x_dev(synth.make_acts(1, k, seed=8))
    buf = torch.zeros(n + 8, device="cuda")
    with pytest.raises(W4a16Error, match="aligned"):
        dec.sk_single_dev("al", x, out=buf[1:n + 1], t=1)          # 4-byte aligned f32 view
    with pytest.raises(W4a16Error, match="aligned"):
        dec.sk_single_static("al", x, out=buf[1:n + 1], t=1)
    xbuf = torch.zeros(k + 8, dtype=torch.float16, device="cuda")
    with pytest.raises(W4a16Error, match="aligned"):
        dec.sk_single_dev("al", xbuf[1:k + 1], t=1)
    assert torch.isfinite(dec.sk_single_dev("al", x, out=buf[4:n + 4], t=1)).all()   # 16-byte aligned view is fine


# Scale / group variants the reference's loader accepts (crates/core/src/w4a16.rs:141-146,225-234): groups of 64
# channels, and bf16 scales -- ordinary ones, and ones far outside the f16 range, which are shifted by a power of
# two at upload and shifted back by the kernels.
@pytest.mark.parametrize("group,bf16,sigma", [(64, False, 0.02), (64, True, 0.02), (32, True, 0.02), (128, True, 0.02),
                                              (32, True, 2e-7), (128, True, 3e5)])
def test_group64_and_bf16_scales(dec, orc, group, bf16, sigma):
    n, k = 512, 1024
    q, s = synth.make_linear(n, k, group, seed=90 + group, sigma=sigma, scale_bf16=bf16)
    dec.upload_lin_g("var", q, s, n, k, group, scale_bf16=bf16)
    assert dec.lin_spec("var") == (n, k, group)
    want = orc.dequant_w4a16(q, s, n, k, group, scale_bf16=bf16)
    got = dec.dequant_lin("var").cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))        # (nibble-8)*scale, bit for bit
    scale = float(np.abs(want).max()) * np.sqrt(k)
    for t in (1, 8, 40):                                                    # decode GEMV and tensor-core GEMM
        x = synth.make_acts(t, k, seed=t)
        y = dec.lin_forward("var", x_dev(x), t).cpu().numpy()
        ref = orc.linear_lane(q, s, x, t, n, k, group, scale_bf16=bf16)
        assert np.abs(y - ref).max() <= max(TOL, 1e-3 * scale) * (1.0 if sigma == 0.02 else np.abs(ref).max() + 1e-30), (t,)
    if sigma == 0.02:
        q2, s2 = dec.unpack_lin("var")                                      # scales come back as f16 values
        assert np.array_equal(q2.cpu().numpy().view(np.uint32), q)
        sf = (s.astype(np.uint32) << 16).view(np.float32) if bf16 else s.view(np.float16).astype(np.float32)
        assert np.array_equal(s2.cpu().numpy().astype(np.float32), sf)
    dec.drop_lin("var")


@pytest.mark.parametrize("n,k,group,bf16,t", [(64, 5120, 128, False, 8), (64, 6144, 128, False, 1), (48, 2048, 32, True, 8),
                                              (32, 768, 64, False, 3), (64, 17408, 128, False, 32)])
def test_lane_mirror_is_bit_identical_to_the_cpu_lane(dec, orc, n, k, group, bf16, t):
    # the reference's gate (crates/server/src/probes/w4a16/gates.rs:108-138): first rows of a linear, x uniform in
    # [-1,1) rounded to f16, every output of the mirror kernel BIT-IDENTICAL to dot_row_w4a16_lane_group
    q, s = synth.make_linear(n, k, group, seed=600 + t, scale_bf16=bf16)
    rng = np.random.default_rng(t)
    x = (rng.random((t, k), dtype=np.float32) * 2 - 1).astype(np.float16).view(np.uint16)
    dec.upload_lin_g("lm", q, s, n, k, group, scale_bf16=bf16)
    got = dec.lin_forward_lane("lm", x_dev(x), t)
    dec.sync()
    want = orc.linear_lane(q, s, x, t, n, k, group, scale_bf16=bf16)
    assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))
    # and the fast kernels agree with it within the gate
    fast = dec.lin_forward("lm", x_dev(x), t)
    dec.sync()
    assert (fast - got).abs().max().item() <= TOL
    dec.drop_lin("lm")


def test_f32_activation_entry_and_multi_segment_above_eight_rows(dec, orc):
    k = 1024
    segs = [("q16", 512), ("k16", 128), ("v16", 144)]
    xs = synth.make_acts(16, k, seed=21)
    x = x_dev(xs)
    for i, (nm, n) in enumerate(segs):
        q, s = synth.make_linear(n, k, 128, seed=70 + i)
        dec.upload_lin_g(nm, q, s, n, k, 128)
    outs = dec.sk_multi_dev([nm for nm, _ in segs], x, t=16)               # batch decode: q|k|v at 16 rows
    for (nm, n), o in zip(segs, outs):
        assert torch.equal(o, dec.lin_forward(nm, x, 16))
    # f32 activations holding f16 values: the same bits as the f16 entry, for the GEMV and the GEMM band
    x32 = x.float()
    for t in (1, 8, 16):
        a = dec.lin_forward_x32("q16", x32[:t].contiguous(), t)
        b = dec.lin_forward("q16", x[:t].contiguous(), t)
        dec.sync()
        assert torch.equal(a, b)


# The reference's batch-decode and speculative-verify chains call the same two entry points with 2..32 rows
# (crates/backend-gpu/src/rawcuda/w4a16_dec/chains.rs:315-507: lin_forward / gemv_multi_t_dev at t = slots or t <= 9 for
# the MTP verify).  Every row count of that band against the lane oracle, through the fused q|k|v call and the single one.
@pytest.mark.parametrize("t", [2, 3, 4, 5, 7, 8, 9, 12, 32])
def test_batch_decode_row_counts_vs_lane_oracle(dec, orc, t):
    k = 1024
    segs = [("bq", 512), ("bk", 128), ("bv", 144)]
    xs = synth.make_acts(t, k, seed=300 + t)
    x = x_dev(xs)
    qs = {}
    for i, (nm, n) in enumerate(segs):
        qs[nm] = synth.make_linear(n, k, 128, seed=310 + i)
        dec.upload_lin_g(nm, *qs[nm], n, k, 128)
    outs = dec.sk_multi_dev([nm for nm, _ in segs], x, t=t)
    dec.sync()
    for (nm, n), o in zip(segs, outs):
        expect = orc.linear_lane(qs[nm][0], qs[nm][1], xs, t, n, k, 128)
        assert np.abs(o.cpu().numpy() - expect).max() <= TOL
        single = dec.lin_forward(nm, x, t)
        dec.sync()
        assert np.abs(single.cpu().numpy() - expect).max() <= TOL


# The row-block form deals the scale groups of K to its warps (16 in the variant for launches whose units are all
# resident at once, 8 otherwise); shapes with fewer groups than warps (the K slices of tensor-parallel shards: o_proj
# over 8 GPUs has K = 768) leave some warps without a group.
@pytest.mark.parametrize("units16", [1, 0])
@pytest.mark.parametrize("n,k", [(512, 768), (272, 128), (1040, 384), (4736, 1152)])
@pytest.mark.parametrize("t", [1, 3, 4])
def test_row_block_form_with_fewer_groups_than_warps(dec, orc, n, k, t, units16):
    q, s = synth.make_linear(n, k, 128, seed=500 + k)
    dec.upload_lin_g("fewg", q, s, n, k, 128)
    xs = synth.make_acts(t, k, seed=510 + t)
    dec.set_tuning("gemv_rowblock_units", units16)
    try:
        y = dec.sk_single_dev("fewg", x_dev(xs), t=t)
        dec.sync()
        assert dec.last_kernel().startswith("gemv_ru_kernel" if units16 else "gemv_rb_kernel")
        expect = orc.linear_lane(q, s, xs, t, n, k, 128)
        assert np.abs(y.cpu().numpy() - expect).max() <= TOL
        y2 = dec.sk_single_dev("fewg", x_dev(xs), t=t)
        dec.sync()
        assert torch.equal(y, y2)
    finally:
        dec.set_tuning("gemv_rowblock_units", 1)


# The 16-warp variant: each warp's first scale group waits in registers, its other groups and the scale words in
# shared memory.  Group counts that do not divide by 16 (K = 5120: 40, K = 2176: 17), exactly 16, one more than 16, an odd
# number of row blocks, every token count, the largest K that fits at two tokens, both output types, guard rows.
@pytest.mark.parametrize("n,k,t", [(7168, 5120, 1), (7168, 5120, 4), (5120, 6144, 2), (1200, 2176, 3), (2064, 2048, 2),
                                   (48, 2176, 1), (9472, 1024, 4), (3584, 4352, 2)])
def test_row_block_16_warp_variant(dec, orc, n, k, t):
    q, s = synth.make_linear(n, k, 128, seed=700 + n % 89)
    dec.upload_lin_g("ru", q, s, n, k, 128)
    xs = synth.make_acts(t, k, seed=710 + t)
    guard = torch.full((t + 1, n), 7.0, device="cuda", dtype=torch.float32)
    y = dec.sk_single_dev("ru", x_dev(xs), t=t, out=guard[:t])
    dec.sync()
    assert dec.last_kernel().startswith("gemv_ru_kernel")
    expect = orc.linear_lane(q, s, xs, t, n, k, 128)
    assert np.abs(y.cpu().numpy() - expect).max() <= TOL
    assert bool((guard[t:] == 7.0).all())
    y16 = dec.sk_single_dev("ru", x_dev(xs), t=t, out_f16=True)
    dec.sync()
    assert torch.equal(y16, y.to(torch.float16))
    # without the variant (the 8-warp kernel, or the K-split form beyond 11264 token-channels): the same sums up to
    # the order in which the parts are added
    dec.set_tuning("gemv_rowblock_units", 0)
    try:
        y8 = dec.sk_single_dev("ru", x_dev(xs), t=t)
        dec.sync()
        assert not dec.last_kernel().startswith("gemv_ru_kernel")
    finally:
        dec.set_tuning("gemv_rowblock_units", 1)
    assert float((y8 - y).abs().max()) <= TOL
    dec.drop_lin("ru")


# More units than resident CTAs (a CTA walks two units, its register ring runs on across the boundary), an odd number
# of row blocks (the last unit holds one), and the 16-row-unit variant for matrices with fewer row blocks than SMs.
@pytest.mark.parametrize("n,k,t", [(12304, 1024, 1), (12304, 1024, 4), (19200, 256, 2), (1200, 2048, 3), (16, 1024, 1)])
def test_row_block_form_units_and_edges(dec, orc, n, k, t):
    q, s = synth.make_linear(n, k, 128, seed=600 + n % 97)
    dec.upload_lin_g("rbu", q, s, n, k, 128)
    xs = synth.make_acts(t, k, seed=610 + t)
    guard = torch.full((t + 1, n), 7.0, device="cuda", dtype=torch.float32)
    y = dec.sk_single_dev("rbu", x_dev(xs), t=t, out=guard[:t])
    dec.sync()
    assert dec.last_kernel().startswith("gemv_rb_kernel" if n > 9472 else "gemv_ru_kernel")
    expect = orc.linear_lane(q, s, xs, t, n, k, 128)
    assert np.abs(y.cpu().numpy() - expect).max() <= TOL
    assert bool((guard[t:] == 7.0).all())
    y16 = dec.sk_single_dev("rbu", x_dev(xs), t=t, out_f16=True)
    dec.sync()
    assert torch.equal(y16, y.to(torch.float16))
    dec.drop_lin("rbu")
