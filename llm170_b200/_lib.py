"""ctypes loader for ``libw4a16_b200.so`` (the C ABI declared in ``include/w4a16_b200.h``).

There is no CPU fallback: if the shared library is missing, loading raises.
"""
from __future__ import annotations

import ctypes as C
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
# W4A16_B200_LIB names another build of the same library (A/B timing of two builds); default: the in-tree one
SO_PATH = os.environ.get("W4A16_B200_LIB") or os.path.join(HERE, "libw4a16_b200.so")
HEADER = os.path.join(os.path.dirname(HERE), "include", "w4a16_b200.h")

_lib = None

_vp, _i, _sz = C.c_void_p, C.c_int, C.c_size_t
_SIGS = {
    "w4a16_dec_new": (_i, [_i, C.POINTER(_vp)]),
    "w4a16_dec_free": (None, [_vp]),
    "w4a16_last_error": (C.c_char_p, [_vp]),
    "w4a16_stream": (_vp, [_vp]),
    "w4a16_sync": (_i, [_vp]),
    "w4a16_kernel_status": (_i, [_vp]),
    "w4a16_debug_timeline": (_i, [_vp, _vp, _i]),
    "w4a16_launch_count": (C.c_ulonglong, [_vp]),
    "w4a16_last_kernel": (C.c_char_p, [_vp]),
    "w4a16_set_tuning": (_i, [_vp, C.c_char_p, _i]),
    "w4a16_check_shapes": (_i, [_sz] * 7),
    "w4a16_upload_lin_g": (_i, [_vp, C.c_char_p, _vp, _sz, _vp, _sz, _i, _i, _i, _i]),
    "w4a16_upload_lin_g_dev": (_i, [_vp, C.c_char_p, _vp, _vp, _i, _i, _i, _i]),
    "w4a16_upload_lin_g_stream": (_i, [_vp, C.c_char_p, _i, _i, _i, _i, _vp, _vp]),
    "w4a16_st_open": (_i, [C.c_char_p, C.POINTER(_vp)]),
    "w4a16_st_close": (None, [_vp]),
    "w4a16_st_error": (C.c_char_p, []),
    "w4a16_st_lin_count": (_i, [_vp]),
    "w4a16_st_lin_at": (_i, [_vp, _i, C.c_char_p, _sz, C.POINTER(_i), C.POINTER(_i), C.POINTER(_i), C.POINTER(_i)]),
    "w4a16_st_lin_tag": (_i, [_vp, C.c_char_p, C.POINTER(C.c_uint64)]),
    "w4a16_upload_lin_st": (_i, [_vp, C.c_char_p, _vp, C.c_char_p]),
    "w4a16_save_lin_cache": (_i, [_vp, C.c_char_p, C.c_char_p, C.c_uint64]),
    "w4a16_load_lin_cache": (_i, [_vp, C.c_char_p, C.c_char_p, C.c_uint64]),
    "w4a16_lin_spec": (_i, [_vp, C.c_char_p, C.POINTER(_i), C.POINTER(_i), C.POINTER(_i)]),
    "w4a16_drop_lin": (_i, [_vp, C.c_char_p]),
    "w4a16_weights_bytes": (_sz, [_vp]),
    "w4a16_unpack_lin": (_i, [_vp, C.c_char_p, _vp, _vp, _vp]),
    "w4a16_dequant_lin": (_i, [_vp, C.c_char_p, _vp, _i, _vp]),
    "w4a16_lin_forward": (_i, [_vp, C.c_char_p, _vp, _vp, _i, _i, _vp]),
    "w4a16_lin_forward_x32": (_i, [_vp, C.c_char_p, _vp, _vp, _i, _i, _vp]),
    "w4a16_lin_forward_lane": (_i, [_vp, C.c_char_p, _vp, _vp, _i, _vp]),
    "w4a16_upload_head": (_i, [_vp, _vp, C.c_size_t, _i, _i]),
    "w4a16_head_spec": (_i, [_vp, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "w4a16_head_unpack": (_i, [_vp, _vp, _vp]),
    "w4a16_head_forward": (_i, [_vp, _vp, _vp, _i, _vp]),
    "w4a16_sk_single_dev": (_i, [_vp, C.c_char_p, _vp, _vp, _i, _i, _vp]),
    "w4a16_sk_single_static": (_i, [_vp, C.c_char_p, _vp, _vp, _i, _i, _vp]),
    "w4a16_tp_create": (_i, [_vp, _i, _i, _i, _vp]),
    "w4a16_tp_connect": (_i, [_vp, _vp]),
    "w4a16_tp_rearm": (_i, [_vp]),
    "w4a16_sk_single_allreduce": (_i, [_vp, C.c_char_p, _vp, _vp, _i, _i, _vp]),
    "w4a16_sk_multi_dev": (_i, [_vp, C.POINTER(C.c_char_p), _i, _vp, C.POINTER(_vp), _i, _i, _vp]),
    "w4a16_lin_forward_host": (_i, [_vp, C.c_char_p, _vp, _vp, _i, _i]),
    "w4a16_gptq4_gemm": (_i, [_vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _vp]),
    "w4a16_set_moe": (_i, [_vp] + [_i] * 7),
    "w4a16_upload_experts": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _i]),
    "w4a16_upload_experts_dev": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _i]),
    "w4a16_moe_topk": (_i, [_vp, _vp, _vp, _vp, _i, _vp]),
    "w4a16_moe_ffn": (_i, [_vp, _i, _vp, _vp, _vp, _i, _i, _vp]),
    "w4a16_capture_begin": (_i, [_vp]),
    "w4a16_capture_end": (_i, [_vp, C.POINTER(_vp)]),
    "w4a16_graph_launch": (_i, [_vp, _vp]),
    "w4a16_graph_destroy": (_i, [_vp, _vp]),
    "w4a16_graph_step_host": (_i, [_vp, _vp, _vp, _vp, _sz, _vp, _vp, _sz]),
}


def declared_symbols() -> list[str]:
    """Every entry point the public header declares."""
    text = open(HEADER).read()
    return sorted(set(re.findall(r"W4A16_API\s+[\w\s\*]+?\b(w4a16_\w+)\s*\(", text)))


FILL_FN = C.CFUNCTYPE(None, _vp, _i, _sz, _vp, _sz)   # w4a16_fill_fn


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(SO_PATH):
            raise RuntimeError(
                f"{SO_PATH} is missing: build it with `python -m llm170_b200.build` "
                "(there is no CPU fallback for the W4A16 path)")
        L = C.CDLL(SO_PATH)
        for name, (res, args) in _SIGS.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib
