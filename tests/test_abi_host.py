"""CPU-side checks of the boundary: the library loads, exports what the header declares, and the
host-side contracts mirror the reference's (crates/backend-gpu/src/rawcuda/gptq4.rs:196-233)."""
import ctypes as C
import os
import subprocess

import pytest

from llm170_b200 import _lib, build
from llm170_b200.gptq4 import check_shapes, kernel_sym
from llm170_b200.w4a16_dec import W4a16Error


@pytest.fixture(scope="module")
def L():
    build.build()
    return _lib.lib()


def test_library_exports_every_declared_symbol(L):
    declared = _lib.declared_symbols()
    assert len(declared) >= 20
    out = subprocess.check_output(["nm", "-D", "--defined-only", _lib.SO_PATH], text=True)
    exported = {ln.split()[-1] for ln in out.splitlines() if " T " in ln}
    missing = [s for s in declared if s not in exported]
    assert not missing, missing
    assert set(declared) == set(_lib._SIGS), set(declared) ^ set(_lib._SIGS)


def test_no_torch_types_in_header():
    text = open(_lib.HEADER).read()
    assert "torch" not in text.lower() and "at::" not in text


def test_every_entry_point_cites_the_reference():
    """Each declaration sits under a comment that cites a reference file (crates/...:line), or says
    in words that the reference has no counterpart."""
    import re
    text = open(_lib.HEADER).read()
    found = 0
    for m in re.finditer(r"/\*(?:[^*]|\*(?!/))*\*/\s*(?:W4A16_API[^;]*;\s*)+", text):
        chunk = m.group(0)
        found += chunk.count("W4A16_API")
        chunk = re.sub(r"\s*\n\s*\*\s*", " ", chunk)   # undo comment line wrapping
        assert re.search(r"crates/[\w/\-.]+:\d+", chunk) or "no counterpart in the reference" in chunk \
            or "reference has no such variant" in chunk, chunk[:200]
    assert found == len(_lib.declared_symbols())


def test_dec_new_fails_loudly_without_gpu(L):
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    h = C.c_void_p()
    assert L.w4a16_dec_new(0, C.byref(h)) != 0
    assert b"no CUDA device" in L.w4a16_last_error(None)
    from llm170_b200.w4a16_dec import W4a16Dec
    with pytest.raises(W4a16Error):
        W4a16Dec(0)


def test_shapes_accept_g128_contract(L):
    # gptq4.rs:199-203
    check_shapes(1, 8 * 640, 8 * 40, 5120, 8, 5120, 128)
    check_shapes(8, 8 * 640, 8 * 40, 8 * 5120, 8, 5120, 128)


def test_shapes_accept_g32_contract(L):
    # gptq4.rs:205-211 (the 8448 case fails there only through the t==1 shared-memory cap, absent here)
    check_shapes(1, 512 * 256, 512 * 64, 2048, 512, 2048, 32)
    check_shapes(8, 512 * 256, 512 * 64, 8 * 2048, 512, 2048, 32)
    check_shapes(1, 8 * 1024, 8 * 256, 8192, 8, 8192, 32)


def test_shapes_reject_bad_rank_and_misalignment(L):
    # gptq4.rs:213-219
    for args in [(1, 8 * 640, 8 * 40, 5120, 8, 5121, 128), (0, 8 * 640, 8 * 40, 0, 8, 5120, 128),
                 (1, 7 * 640, 8 * 40, 5120, 8, 5120, 128), (1, 8 * 640, 8 * 40, 5120, 8, 5120, 64)]:
        with pytest.raises(W4a16Error):
            check_shapes(*args)


def test_kernel_sym_selects_variants():
    # gptq4.rs:228-233, adapted: the names are the kernel instantiations this library launches; group 64 is
    # served by the group-32 kernels (its scales are stored twice), other groups are rejected
    assert kernel_sym(False, 128, False) == "gemv_sk_kernel<128,true>"
    assert kernel_sym(True, 128, False) == "gemm_w4a16_tc_kernel<128,1>"
    assert kernel_sym(False, 32, True) == "gemv_sk_kernel<32,true>"
    assert kernel_sym(True, 64, False) == "gemm_w4a16_tc_kernel<32,1>"
    with pytest.raises(W4a16Error):
        kernel_sym(True, 16, False)


def test_layout_word_index_is_a_bijection():
    """Python restatement of csrc/layout.cuh word_index: every (row,k) maps to a distinct nibble slot."""
    import numpy as np
    n, k = 32, 128
    seen = set()
    for row in range(n):
        for kk in range(k):
            rb, rr = divmod(row, 16)
            g, hi = rr & 7, rr >> 3
            kb, kr = divmod(kk, 64)
            p, t, h, e = kr >> 5, (kr >> 3) & 3, (kr >> 2) & 1, kr & 3
            pos = (((e & 1) << 2) | (e & 2)) + hi
            w = (kb * (n // 16) + rb) * 128 + (4 * g + t) * 4 + 2 * p + h
            seen.add((w, pos))
    assert len(seen) == n * k and max(w for w, _ in seen) == n * k // 8 - 1
