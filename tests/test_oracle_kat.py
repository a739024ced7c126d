"""Pins the CPU oracle to the reference's own known-answer tests for the W4A16 path.

Every test restates one reference test (cited by file:line) with the same seeds,
generators and assertions; none reads the reference tree at run time.
"""
import math

import numpy as np

M64 = (1 << 64) - 1


def to_f16_ref(v: float) -> int:
    """The test-local f32->f16 of crates/core/src/quant/lane.rs:76-97 (round half up, flush tiny)."""
    b = int(np.float32(v).view(np.uint32))
    sign = (b >> 16) & 0x8000
    exp = ((b >> 23) & 0xFF) - 127 + 15
    man = b & 0x7FFFFF
    if exp <= 0:
        return sign
    if exp >= 31:
        return sign | 0x7C00
    m = (man >> 13) + ((man >> 12) & 1)
    if m & 0x400:
        m, exp = m & 0x3FF, exp + 1
    return sign | (exp << 10) | m


class XorShift:
    """xorshift64 used by crates/core/src/quant/lane.rs:101-108."""

    def __init__(self, seed):
        self.s = seed

    def __call__(self):
        s = self.s
        s ^= (s << 13) & M64
        s ^= s >> 7
        s ^= (s << 17) & M64
        self.s = s
        return s


def f32(v):
    return np.float32(v)


def test_lane_matches_scalar(orc):
    # crates/core/src/quant/lane.rs:99-138
    k = 256
    rnd = XorShift(0x9E3779B9)
    qrow = np.array([rnd() & 0xFFFFFFFF for _ in range(k // 8)], np.uint32)
    zrow = np.array([rnd() % 16 for _ in range(k // 128)], np.uint32)
    srow = np.array([to_f16_ref(f32(0.25) + f32(rnd() % 100) / f32(400.0)) for _ in range(k // 128)], np.uint16)
    x = np.array([to_f16_ref(f32(rnd() % 2000) / f32(1000.0) - f32(1.0)) for _ in range(k)], np.uint16)
    got = orc.dot_row_w4a16_lane(qrow, zrow, srow, x)
    want = 0.0
    for i in range(k):
        g = i // 128
        q = (int(qrow[i // 8]) >> (4 * (i % 8))) & 0xF
        w = f32(q - int(zrow[g])) * f32(orc.half_to_f32(int(srow[g])))
        want += float(f32(w) * f32(orc.half_to_f32(int(x[i]))))
    rel = abs(float(got) - want) / max(abs(want), 1e-9)
    assert rel < 1e-6, (got, want, rel)


def test_f16b_is_ieee_half(orc):
    # crates/core/src/quant/lane.rs:141-145
    assert orc.half_to_f32(0x3C00) == 1.0
    assert orc.half_to_f32(0x3800) == 0.5
    assert orc.half_to_f32(0xC000) == -2.0


def test_half_to_f32_all_patterns_match_numpy(orc):
    # crates/core/src/quant/deq.rs:4-27 is IEEE: compare all 65536 patterns with numpy's half.
    h = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    want = h.view(np.float16).astype(np.float32).view(np.uint32)
    got = np.array([np.float32(orc.half_to_f32(int(v))).view(np.uint32) for v in h[::7]], np.uint32)
    w7 = want[::7]
    nan = np.isnan(w7.view(np.float32))
    assert np.array_equal(got[~nan], w7[~nan])
    assert np.all(np.isnan(got[nan].view(np.float32)))


def test_f32_to_f16_rne_matches_numpy(orc):
    # crates/backend-gpu/src/rawcuda/w4a16_dec/mod.rs:187-219 is round-to-nearest-even.
    rng = np.random.default_rng(7)
    v = np.concatenate([
        rng.standard_normal(4000).astype(np.float32),
        (rng.standard_normal(2000) * 1e-6).astype(np.float32),
        (rng.standard_normal(500) * 7e4).astype(np.float32),
        np.array([0.0, -0.0, 65504.0, 65520.0, 65519.9, 2.0 ** -24, 2.0 ** -25, 3 * 2.0 ** -26,
                  np.inf, -np.inf, 1.00048828125], np.float32),
    ])
    with np.errstate(over="ignore"):
        want = v.astype(np.float16).view(np.uint16)
    got = np.array([orc.f32_to_f16(float(t)) for t in v], np.uint16)
    assert np.array_equal(got, want)
    assert orc.f32_to_f16(float("nan")) & 0x7E00 == 0x7E00


def test_lane_g32_bf16_scale(orc):
    # crates/core/src/quant/lane.rs:148-183  (bit equality against the spelled-out lane loop)
    k = 256
    rnd = XorShift(0x12345678)
    qrow = np.array([rnd() & 0xFFFFFFFF for _ in range(k // 8)], np.uint32)
    zrow = np.array([rnd() % 16 for _ in range(k // 32)], np.uint32)
    srow = []
    for _ in range(k // 32):
        v = f32(0.25) + f32(rnd() % 100) / f32(400.0)
        srow.append(orc.bf16_to_f32(int(np.float32(v).view(np.uint32)) >> 16))
    srow = np.array(srow, np.float32)
    x = np.array([to_f16_ref(f32(rnd() % 2000) / f32(1000.0) - f32(1.0)) for _ in range(k)], np.uint16)
    got = orc.dot_row_w4a16_lane_group(qrow, zrow, srow, x, 32)
    xf = x.view(np.float16).astype(np.float32)
    lanes = np.zeros(64, np.float64)
    for l in range(64):
        acc = f32(0.0)
        for i in range(l, k, 64):
            g = i // 32
            q = (int(qrow[i >> 3]) >> (4 * (i & 7))) & 0xF
            w = f32(f32(q - int(zrow[g])) * srow[g])
            acc = f32(acc + f32(w * xf[i]))
        lanes[l] = float(acc)
    a = lanes.copy()
    a[:32] += a[32:]
    for off in (16, 8, 4, 2, 1):
        a[:off] += a[off:2 * off]
    assert np.float32(a[0]).view(np.uint32) == np.float32(got).view(np.uint32)
    assert orc.tree64(lanes) == a[0]


def test_sym_zp8_center(orc):
    # crates/core/src/quant/lane.rs:186-193
    k = 128
    qrow = np.full(k // 8, 0x88888888, np.uint32)
    got = orc.dot_row_w4a16_lane(qrow, np.array([8], np.uint32), np.array([to_f16_ref(0.5)], np.uint16),
                                 np.full(k, to_f16_ref(1.0), np.uint16))
    assert got == 0.0


def test_lane_rejects_unaligned_k(orc):
    # crates/core/src/quant/lane.rs:51-54 (assert on group alignment)
    import pytest
    with pytest.raises(ValueError):
        orc.lane_parts_scale(np.zeros(12, np.uint32), np.zeros(3, np.uint32), np.zeros(3, np.float32),
                             np.zeros(96, np.uint16), 64)
    with pytest.raises(ValueError):
        orc.lane_parts_scale(np.zeros(6, np.uint32), np.zeros(3, np.uint32), np.zeros(3, np.float32),
                             np.zeros(48, np.uint16), 16)


def test_repack_roundtrip(orc):
    # crates/core/src/marlin.rs:107-122
    n, k = 128, 64
    seed = 0x123456789ABCDEF0
    q = np.zeros(n * (k // 8), np.uint32)
    for i in range(q.size):
        seed = (seed * 6364136223846793005 + 1442695040888963407) & M64
        q[i] = seed >> 32
    packed = orc.marlin_repack_q(q, n, k)
    assert packed.size == (k // 16) * (n // 64) * 128
    assert np.array_equal(orc.marlin_unrepack_q(packed, n, k), q)


def test_repack_contract(orc):
    # crates/core/src/marlin.rs:3-13
    import pytest
    with pytest.raises(ValueError):
        orc.marlin_repack_q(np.zeros(64 * 3, np.uint32), 64, 24)
    with pytest.raises(ValueError):
        orc.marlin_repack_q(np.zeros(32 * 2, np.uint32), 32, 16)
    with pytest.raises(ValueError):
        orc.marlin_repack_q(np.zeros(5, np.uint32), 64, 16)


def test_scale_perm_roundtrip(orc):
    # crates/core/src/marlin.rs:124-131
    n, k, gs = 64, 128, 128
    s = np.arange(n * (k // gs), dtype=np.float32)
    out = orc.marlin_permute_scales(s, n, k, gs)
    for p in range(64):
        assert out[p] == s[p // 8 + 8 * (p % 8)]


def test_split_dequant_row_g128_f16(orc):
    # crates/core/src/matmul/cpu.rs:228-250
    k, group = 256, 128
    word = sum((j & 0xF) << (4 * j) for j in range(8))
    q = np.full(k // 8, word, np.uint32).view(np.uint8)
    s = np.array([0x3C00, 0x3800], np.uint16).view(np.uint8)
    out = orc.dequant_row_w4a16_split(q, s, 0, k, group, False)
    for i, v in enumerate(out):
        assert v == np.float32((i % 8) - 8) * (1.0 if i < 128 else 0.5), i


def test_split_dequant_row_g32_bf16(orc):
    # crates/core/src/matmul/cpu.rs:252-271
    k, group = 64, 32
    word = sum(((7 - j) & 0xF) << (4 * j) for j in range(8))
    q = np.full(k // 8, word, np.uint32).view(np.uint8)
    s = np.array([0x3F80, 0x3F80], np.uint16).view(np.uint8)
    out = orc.dequant_row_w4a16_split(q, s, 0, k, group, True)
    for i, v in enumerate(out):
        assert v == np.float32((7 - (i % 8)) - 8), i


def test_select_topk_renormalizes_and_orders(orc):
    # crates/core/src/qwen35/stages/moe.rs:135-146 and crates/backend-gpu/src/rawcuda/w4a16_dec/tests.rs:5-15
    sel = orc.select_topk([2.0, 1.0, 0.5, -1.0], 2)
    assert [e for e, _ in sel] == [0, 1]
    assert sel[0][1] > sel[1][1]
    assert abs(float(sel[0][1] + sel[1][1]) - 1.0) < 1e-6
    assert abs(float(sel[0][1] / sel[1][1]) - math.e) < 1e-4


def test_select_topk_tie_breaks_low_index(orc):
    # crates/core/src/qwen35/stages/moe.rs:148-155 and crates/backend-gpu/src/rawcuda/w4a16_dec/tests.rs:16-18
    sel = orc.select_topk([1.0, 1.0, 1.0], 2)
    assert [e for e, _ in sel] == [0, 1]
    assert abs(float(sel[0][1] + sel[1][1]) - 1.0) < 1e-6


def test_decode_selfcheck_expectation(orc):
    # crates/backend-gpu/src/rawcuda/w4a16_dec/probe.rs:1291-1308: scale = x = 1.0 -> y = sum(nib-8) exactly.
    n, k = 256, 512
    i = np.arange(n * k // 8, dtype=np.uint64)
    q = (((i * 0x9E3779B9) & 0xFFFFFFFF) ^ 0x12345678).astype(np.uint32).reshape(n, k // 8)
    s = np.full((n, k // 128), 0x3C00, np.uint16)
    x = np.full((1, k), 0x3C00, np.uint16)
    y = orc.linear_lane(q, s, x, 1, n, k, 128)
    nib = ((q[:, :, None] >> (4 * np.arange(8, dtype=np.uint32))) & 0xF).astype(np.int64) - 8
    assert np.array_equal(y[0], nib.reshape(n, -1).sum(axis=1).astype(np.float32))


def test_marlin_selfcheck_expectation(orc):
    # crates/server/src/probes/w4a16/gpu/bench.rs:77-121: nib=(7k+3n)%16, power-of-two scales and x
    # -> the f64 expectation is exact and the lane dot must equal it bit for bit.
    t, k, n = 16, 256, 128
    kk, nn = np.meshgrid(np.arange(k), np.arange(n))
    nib = ((kk * 7 + nn * 3) % 16).astype(np.uint32)
    q = np.bitwise_or.reduce(nib.reshape(n, k // 8, 8) << (4 * np.arange(8, dtype=np.uint32)), axis=2).astype(np.uint32)
    s = np.array([[(15 - ((r + g) % 5)) << 10 for g in range(k // 128)] for r in range(n)], np.uint16)
    i = np.arange(t * k)
    x = ((15 - ((i // k + (i % k) // 8) % 4)) << 10).astype(np.uint16).reshape(t, k)
    sf = s.view(np.float16).astype(np.float64)
    xf = x.view(np.float16).astype(np.float64)
    w = (nib.astype(np.float64) - 8.0) * np.repeat(sf, 128, axis=1)
    expect = (xf @ w.T).astype(np.float32)
    got = orc.linear_lane(q, s, x, t, n, k, 128)
    assert np.array_equal(got.view(np.uint32), expect.view(np.uint32))


def test_marlin_selfcheck32_expectation(orc):
    # crates/server/src/probes/w4a16/gpu/bench.rs:123-166: g32, bf16-coded 2^-j scales, x = 1.
    t, k, n = 4, 128, 64
    kk, nn = np.meshgrid(np.arange(k), np.arange(n))
    nib = ((kk * 7 + nn * 3) % 16).astype(np.uint32)
    q = np.bitwise_or.reduce(nib.reshape(n, k // 8, 8) << (4 * np.arange(8, dtype=np.uint32)), axis=2).astype(np.uint32)
    s = np.array([[(127 - ((r + g) % 5)) << 7 for g in range(k // 32)] for r in range(n)], np.uint16)
    x = np.full((t, k), 0x3C00, np.uint16)
    j = (nn + kk // 32) % 5
    expect = ((nib.astype(np.float64) - 8.0) * np.power(2.0, -j)).sum(axis=1).astype(np.float32)
    got = orc.linear_lane(q, s, x, t, n, k, 32, scale_bf16=True)
    for r in range(t):
        assert np.array_equal(got[r].view(np.uint32), expect.view(np.uint32))


def test_gate_inputs_lane_group_equals_linear(orc):
    # crates/server/src/probes/w4a16/gates.rs:108-126: SplitMix64 x in [-1,1) -> f16, z=8, per-row lane dot.
    def splitmix(seed):
        s = seed
        while True:
            s = (s + 0x9E3779B97F4A7C15) & M64
            z = s
            z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M64
            z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M64
            yield z ^ (z >> 31)
    from llm170_b200 import synth
    n, k, group, t = 4, 512, 128, 8
    q, s = synth.make_linear(n, k, group, seed=11)
    gen = splitmix(1 ^ (n << 32) ^ k)
    x = np.array([orc.f32_to_f16(float(np.float32(np.float32(next(gen) >> 40) / np.float32(1 << 24)) * np.float32(2.0) - np.float32(1.0)))
                  for _ in range(t * k)], np.uint16).reshape(t, k)
    full = orc.linear_lane(q, s, x, t, n, k, group)
    z8 = np.full(k // group, 8, np.uint32)
    sf = s.view(np.float16).astype(np.float32)
    for ti in range(t):
        for o in range(n):
            want = orc.dot_row_w4a16_lane_group(q[o], z8, sf[o], x[ti], group)
            assert np.float32(want).view(np.uint32) == full[ti, o].view(np.uint32)


def test_linear_rows_subset_and_threads(orc):
    from llm170_b200 import synth
    n, k = 96, 256
    q, s = synth.make_linear(n, k, 128, seed=3)
    x = synth.make_acts(3, k, seed=3)
    a = orc.linear_lane(q, s, x, 3, n, k, 128, nthreads=1)
    b = orc.linear_lane(q, s, x, 3, n, k, 128, nthreads=5)
    assert np.array_equal(a, b)
    c = orc.linear_lane(q, s, x, 3, n, k, 128, rows=(10, 50))
    assert np.array_equal(c[:, 10:50], a[:, 10:50]) and not c[:, :10].any() and not c[:, 50:].any()


def _f16_round(orc, v):
    """f32 array -> f16 values (as f32), element by element through the pinned orc.f32_to_f16."""
    flat = np.asarray(v, np.float32).ravel()
    bits = np.array([orc.f32_to_f16(float(e)) for e in flat], np.uint16)
    return np.array([orc.half_to_f32(int(b)) for b in bits], np.float32).reshape(np.shape(v)), bits.reshape(np.shape(v))


def test_moe_ffn_equals_stepwise_chain_of_pinned_primitives(orc):
    """The resident MoE chain of crates/backend-gpu/src/rawcuda/w4a16_dec/kernels/marlin_moe.rs:290-422, restated
    a second time, token by token and row by row, from primitives that the known-answer tests above pin
    (select_topk, dot_row_w4a16_lane_group, half_to_f32, f32_to_f16): grouped matmul 1 -> f16, silu(gate)*up in
    f32 -> f16 (assets/moe.cu:1649-1660), grouped matmul 2 -> f16, times the f16 routing weight -> f16
    (assets/marlin_moe/marlin_template.h:1515-1524), f32 sum over k in slot order (assets/moe.cu:1662-1674).
    Weights, scales and activations are powers of two (the recipe of probes/w4a16/gpu/bench.rs:123-166), so
    matmul 1 is exact whatever the summation order.  oracle.moe_ffn must agree bit for bit.  The reference holds
    no known answer for the whole chain; this composition is the strongest pin available for it."""
    n_exp, top_k, f, h, group, t = 4, 2, 64, 64, 32, 5
    def pow2_linear(n, k, salt):
        kk, nn = np.meshgrid(np.arange(k), np.arange(n))
        nib = ((kk * 7 + nn * 3 + salt) % 16).astype(np.uint32)
        q = np.bitwise_or.reduce(nib.reshape(n, k // 8, 8) << (4 * np.arange(8, dtype=np.uint32)), axis=2).astype(np.uint32)
        s = np.array([[(12 - ((r + g + salt) % 4)) << 10 for g in range(k // group)] for r in range(n)], np.uint16)
        return q, s
    w13 = [pow2_linear(2 * f, h, e) for e in range(n_exp)]
    w2 = [pow2_linear(h, f, 5 + e) for e in range(n_exp)]
    w13_q, w13_s = np.stack([a for a, _ in w13]), np.stack([b for _, b in w13])
    w2_q, w2_s = np.stack([a for a, _ in w2]), np.stack([b for _, b in w2])
    i = np.arange(t * h)
    x = ((13 - ((i // h + (i % h) // 8) % 3)) << 10).astype(np.uint16).reshape(t, h)
    x[:, ::5] ^= 0x8000                                    # some negative activations
    rng = np.random.Generator(np.random.PCG64(11))
    logits = rng.standard_normal((t, n_exp)).astype(np.float32)

    def lin_row(q_row, s_row, xv, k):
        z = np.full(k // group, 8, np.uint32)
        sf = np.array([orc.half_to_f32(int(b)) for b in s_row], np.float32)
        return orc.dot_row_w4a16_lane_group(q_row, z, sf, xv, group)

    want = np.zeros((t, h), np.float32)
    for ti in range(t):
        acc = np.zeros(h, np.float32)
        for e, wgt in orc.select_topk(logits[ti], top_k):
            c13 = np.array([lin_row(w13_q[e][r], w13_s[e][r], x[ti], h) for r in range(2 * f)], np.float32)
            c13, _ = _f16_round(orc, c13)
            g, u = c13[:f], c13[f:]
            act32 = (g / (np.float32(1.0) + np.exp(-g, dtype=np.float32))) * u
            _, act_bits = _f16_round(orc, act32)
            c2 = np.array([lin_row(w2_q[e][r], w2_s[e][r], act_bits, f) for r in range(h)], np.float32)
            c2h, _ = _f16_round(orc, c2)
            wh, _ = _f16_round(orc, np.float32(wgt))
            contrib, _ = _f16_round(orc, c2h * wh)           # product of two f16 values: exact in f32, one rounding
            acc = acc + contrib
        want[ti] = acc
    got = orc.moe_ffn(x, logits, w13_q, w13_s, w2_q, w2_s, top_k, group)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # matmul 1 is exact for these inputs: check one expert against plain f64 arithmetic as well
    e = 1
    nib = ((w13_q[e][:, :, None] >> (4 * np.arange(8, dtype=np.uint32))) & 0xF).astype(np.float64).reshape(2 * f, h) - 8
    wd = nib * np.repeat(w13_s[e].view(np.float16).astype(np.float64), group, axis=1)
    exact = (x.view(np.float16).astype(np.float64) @ wd.T).astype(np.float32)
    assert np.array_equal(orc.linear_lane(w13_q[e], w13_s[e], x, t, 2 * f, h, group), exact)


# ---- int8 lm-head (no known-answer test of its own in the reference: checked on inputs whose answer is forced) ----
def test_head_quant_recipe_on_forced_values(orc):
    # crates/backend-gpu/src/rawcuda/w4a16_dec/upload.rs:1495-1516: scale = absmax/127 (1 for a zero row),
    # q = round-half-away(v/scale) clamped to +-127
    def bf16(v):
        return (np.asarray(v, np.float32).view(np.uint32) >> 16).astype(np.uint16)   # values below are exact in bf16
    rows = np.zeros((3, 8), np.float32)
    rows[0] = [127.0, 0.5, 1.5, -2.5, -0.5, 63.5, -126.5, 3.0]     # scale 1: ties go away from zero
    rows[2] = [0.25, -0.125, 0.0, 0.0625, -0.25, 0.125, 0.0, 0.0]  # scale 0.25/127
    q, sc = orc.head_quant(bf16(rows), 3, 8)
    assert sc.tolist() == [1.0, 1.0, np.float32(0.25) / np.float32(127.0)]
    assert q[0].tolist() == [127, 1, 2, -3, -1, 64, -127, 3]
    assert not q[1].any()
    assert q[2].tolist() == [127, -64, 0, 32, -127, 64, 0, 0]      # 63.5 -> 64, 31.75 -> 32


def test_head_gemv_lane_order_exact_and_random(orc):
    # exact case: integers times powers of two, every partial sum exact -> equals float64 arithmetic
    n, k = 8, 512
    q = ((np.arange(n * k).reshape(n, k) * 11) % 255 - 127).astype(np.int8)
    sc = (2.0 ** -(np.arange(n) % 4)).astype(np.float32)
    x = (2.0 ** ((np.arange(2 * k) % 7) - 3)).astype(np.float32).reshape(2, k)
    y = orc.head_gemv_i8(q, sc, x, 2)
    assert np.array_equal(y, ((x.astype(np.float64) @ q.astype(np.float64).T) * sc).astype(np.float32))
    # random case: the lane order stays within f32 rounding of the exact sum
    rng = np.random.default_rng(3)
    x = rng.standard_normal((1, k)).astype(np.float32)
    y = orc.head_gemv_i8(q, sc, x, 1)
    exact = (x.astype(np.float64) @ q.astype(np.float64).T) * sc
    assert np.abs(y - exact).max() <= 1e-6 * (np.abs(x).astype(np.float64) @ np.abs(q).astype(np.float64).T * sc).max()
