"""GPU tests of the load path: checkpoint -> streamed, chunk-wise re-tiling -> resident tiles -> tile cache file ->
reload with plain copies.  The tiles of every route must be bit-identical, and dequantise to the oracle's values."""
import os

import numpy as np
import pytest
import torch

from llm170_b200 import synth
from test_loader_host import TINY, read_st

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dec():
    from llm170_b200.w4a16_dec import W4a16Dec
    d = W4a16Dec(0)
    yield d
    d.close()


@pytest.mark.parametrize("sub", ["dense", "experts"])
def test_checkpoint_directory_to_device_and_cache(dec, orc, tmp_path, sub):
    from llm170_b200.w4a16_model import W4a16Model
    model = W4a16Model(os.path.join(TINY, sub))
    raw = read_st(os.path.join(TINY, sub, "model.safetensors"))
    cache = str(tmp_path / "cache")
    how = model.upload_all(dec, cache_dir=cache)
    assert set(how.values()) == {"checkpoint"}
    deq = {}
    for base, (n, k, g, bf) in model.lins.items():
        assert dec.lin_spec(base) == (n, k, g)
        q = np.frombuffer(raw[base + ".weight_packed"][2], "<u4").reshape(n, k // 8)
        s = np.frombuffer(raw[base + ".weight_scale"][2], "<u2").reshape(n, k // g)
        want = orc.dequant_w4a16(q, s, n, k, g, scale_bf16=bf)
        got = dec.dequant_lin(base).cpu().numpy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        x = synth.make_acts(3, k, seed=k)
        y = dec.lin_forward(base, torch.from_numpy(x.view(np.float16).copy()).cuda(), 3).cpu().numpy()
        assert np.abs(y - orc.linear_lane(q, s, x, 3, n, k, g, scale_bf16=bf)).max() <= 2e-3
        deq[base] = (got, y)
        dec.drop_lin(base)
    # second load: every linear comes from its cache file, and is the same bits
    how = model.upload_all(dec, cache_dir=cache)
    assert set(how.values()) == {"cache"}
    for base, (n, k, g, bf) in model.lins.items():
        assert dec.lin_spec(base) == (n, k, g)
        assert np.array_equal(dec.dequant_lin(base).cpu().numpy(), deq[base][0])
        x = synth.make_acts(3, k, seed=k)
        y = dec.lin_forward(base, torch.from_numpy(x.view(np.float16).copy()).cuda(), 3).cpu().numpy()
        assert np.array_equal(y, deq[base][1])
    # a cache file made from other tensors is refused (stale), and rebuilt
    from llm170_b200.w4a16_dec import W4a16Error
    first = sorted(model.lins)[0]
    path = os.path.join(cache, first.replace("/", "_") + ".w4t64")
    with pytest.raises(W4a16Error, match="stale"):
        dec.load_lin_cache("x", path, model.st.tag(first) ^ 1)
    blob = bytearray(open(path, "rb").read())
    blob[8] ^= 0xFF                                  # another layout version
    open(path, "wb").write(blob)
    with pytest.raises(W4a16Error, match="version"):
        dec.load_lin_cache("x", path, model.st.tag(first))
    assert model.upload_all(dec, cache_dir=cache)[first] == "checkpoint"
    model.close()


@pytest.mark.parametrize("n,k,group,bf16", [(4096, 5120, 128, False), (1536, 2048, 32, True), (48, 17408, 64, False)])
def test_streamed_upload_equals_one_shot_upload(dec, n, k, group, bf16):
    # chunked re-tiling (several 8 MiB row chunks for the first shape) against the whole-tensor device repack
    q, s = synth.make_linear(n, k, group, seed=n + k, scale_bf16=bf16)
    dec.upload_lin_g_dev("whole", torch.from_numpy(q.view(np.int32)).cuda(), torch.from_numpy(s.view(np.int16)).cuda(), n, k,
                         group, scale_bf16=bf16)
    want = dec.dequant_lin("whole", f16=True)
    calls = []

    def fill(which, off, buf):
        src = (q if which == 0 else s).view(np.uint8).ravel()
        buf[:] = src[off:off + len(buf)].tobytes()
        calls.append((which, off, len(buf)))
    dec.upload_lin_g_stream("chunked", n, k, group, bf16, fill)
    assert torch.equal(dec.dequant_lin("chunked", f16=True), want)
    assert max(c[2] for c in calls) <= 8 << 20                          # nothing larger than a chunk was asked for
    assert sum(c[2] for c in calls if c[0] == 0) == q.nbytes
    dec.upload_lin_g("slice", q, s, n, k, group, scale_bf16=bf16)      # the host-slice entry rides on the same path
    assert torch.equal(dec.dequant_lin("slice", f16=True), want)
    x = torch.from_numpy(synth.make_acts(2, k, seed=3).view(np.float16).copy()).cuda()
    assert torch.equal(dec.lin_forward("chunked", x, 2), dec.lin_forward("whole", x, 2))
    for nm in ("whole", "chunked", "slice"):
        dec.drop_lin(nm)
