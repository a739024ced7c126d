"""GPU parity of the int8 lm-head (quantiser and GEMV) through the C ABI.

The quantiser must reproduce the reference's host recipe bit for bit (crates/backend-gpu/src/rawcuda/w4a16_dec/
upload.rs:1472-1518).  The GEMV is compared with the CPU restatement of the reference's kernel
(crates/backend-gpu/src/rawcuda/assets/head.cu:100-225: 64 f32 lane sums, f64 tree); the two add the same exact
products in different orders, so the gate is relative to the sum of the products' magnitudes:
|y - oracle| <= 1e-5 * sum_k |q x| * scale  (two f32 accumulations of k terms in different orders; measured up to 4e-6)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
REL = 1e-5


@pytest.fixture(scope="module")
def dec():
    from llm170_b200.w4a16_dec import W4a16Dec
    d = W4a16Dec(0)
    yield d
    d.close()


def bf16_of(w32):
    """f32 -> bf16 bit patterns, round to nearest even (what a checkpoint holds)."""
    u = np.ascontiguousarray(w32, np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def make_head(n, k, seed):
    rng = np.random.default_rng(seed)
    w = bf16_of(rng.standard_normal((n, k)).astype(np.float32) * 0.02)
    return w


def test_quantiser_is_bit_identical_to_the_host_recipe(dec, orc):
    n, k = 300, 512
    w = make_head(n, k, 5)
    w[7, :] = 0                                           # a zero row: scale 1, all zeros
    # a row whose scale is exactly 1 and whose values sit on rounding ties (half away from zero)
    ties = np.array([127.0, 0.5, 1.5, -2.5, -0.5, 63.5, -126.5, 3.0], np.float32)
    w[11, :] = bf16_of(np.resize(ties, k))
    dec.upload_head(w, n, k)
    q, sc = dec.head_unpack()
    q_o, sc_o = orc.head_quant(w, n, k)
    assert np.array_equal(sc.view(np.uint32), sc_o.view(np.uint32))
    assert np.array_equal(q, q_o)
    assert sc[7] == 1.0 and not q[7].any()
    assert q[11, :8].tolist() == [127, 1, 2, -3, -1, 64, -127, 3]
    assert dec.head_spec() == (n, k)


@pytest.mark.parametrize("n,k,t", [(1000, 256, 1), (4096, 2048, 1), (2056, 5120, 1), (1000, 2048, 2), (777, 1024, 5),
                                   (4096, 2048, 8), (1000, 2048, 9), (2048, 5120, 16)])
def test_head_gemv_vs_lane_order_oracle(dec, orc, n, k, t):
    w = make_head(n, k, 100 + t)
    dec.upload_head(w, n, k)
    q, sc = orc.head_quant(w, n, k)
    rng = np.random.default_rng(200 + t)
    x = rng.standard_normal((t, k)).astype(np.float32)
    x[0, :8] = [0.0, 1e-6, -3e-5, 250.0, -1000.0, 0.3333333, 7.0, -0.001]   # small, large and plain values
    guard = torch.full((t + 1, n), 7.0, device="cuda", dtype=torch.float32)
    y = dec.head_forward(torch.from_numpy(x).cuda(), t, out=guard[:t])
    dec.sync()
    expect = orc.head_gemv_i8(q, sc, x, t)
    bound = REL * (np.abs(x).astype(np.float64) @ np.abs(q).astype(np.float64).T) * sc
    err = np.abs(y.cpu().numpy().astype(np.float64) - expect)
    assert (err <= bound + 1e-30).all(), float((err / (bound + 1e-30)).max())
    assert bool((guard[t:] == 7.0).all())
    # the same call twice gives the same bits
    y2 = dec.head_forward(torch.from_numpy(x).cuda(), t)
    dec.sync()
    assert torch.equal(y, y2)


def test_exact_case_matches_integer_arithmetic(dec):
    # power-of-two activations and small integers: every partial sum is exact in f32 whatever the order
    n, k = 64, 256
    ints = ((np.arange(n * k).reshape(n, k) * 7) % 255 - 127).astype(np.float32)
    ints[:, 0] = 127.0                                    # absmax 127 -> scale exactly 1
    w = bf16_of(ints)
    dec.upload_head(w, n, k)
    q, sc = dec.head_unpack()
    assert np.array_equal(q.astype(np.float32), ints) and (sc == 1.0).all()
    x = (2.0 ** ((np.arange(k) % 5) - 2)).astype(np.float32)[None, :]
    y = dec.head_forward(torch.from_numpy(x).cuda(), 1)
    dec.sync()
    assert np.array_equal(y.cpu().numpy()[0], (ints.astype(np.float64) @ x[0].astype(np.float64)).astype(np.float32))


def test_contract_errors():
    from llm170_b200.w4a16_dec import W4a16Dec, W4a16Error
    d = W4a16Dec(0)
    try:
        with pytest.raises(W4a16Error, match="no lm-head"):
            d.head_forward(torch.zeros(64, device="cuda"), 1)
        with pytest.raises(W4a16Error, match="multiple of 64"):
            d.upload_head(np.zeros((16, 100), np.uint16), 16, 100)
        d.upload_head(np.zeros((16, 128), np.uint16), 16, 128)
        with pytest.raises(W4a16Error, match="1..16"):
            d.head_forward(torch.zeros(17 * 128, device="cuda"), 17)
    finally:
        d.close()
