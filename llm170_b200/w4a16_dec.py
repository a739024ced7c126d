"""Host-side mirror of the reference's ``W4a16Dec`` linear call sites, over the C ABI.

Method names, argument meaning and error behaviour follow
crates/backend-gpu/src/rawcuda/w4a16_dec/{upload.rs,kernels/mod.rs,kernels/decode.rs}: every
method raises ``W4a16Error`` with the library's message where the reference returns
``Err(String)``.  Device buffers are ``torch`` CUDA tensors (plumbing only); the work runs in
``libw4a16_b200.so`` on the caller's current CUDA stream.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _lib

OUT_F32, OUT_F16 = 0, 1


class W4a16Error(RuntimeError):
    pass


def _cur_stream() -> int:
    """torch's current stream as a cudaStream_t.  torch's default stream has the handle 0, which the
    C ABI reads as "use the decoder's own stream"; 1 is cudaStreamLegacy, the explicit name of that
    same default stream, so work stays ordered with the caller's torch ops."""
    h = int(torch.cuda.current_stream().cuda_stream)
    return h if h != 0 else 1


class W4a16Dec:
    def __init__(self, device: int = 0):
        if not torch.cuda.is_available():
            raise W4a16Error("W4a16Dec needs a CUDA device (no CPU fallback exists)")
        self._L = _lib.lib()
        self.device = device
        torch.cuda.set_device(device)
        h = C.c_void_p()
        if self._L.w4a16_dec_new(device, C.byref(h)) != 0:
            raise W4a16Error(self._L.w4a16_last_error(None).decode())
        self._h = h

    # -- plumbing ---------------------------------------------------------------------------
    def close(self):
        if getattr(self, "_h", None):
            self._L.w4a16_dec_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _ck(self, rc: int):
        if rc != 0:
            raise W4a16Error(self._L.w4a16_last_error(self._h).decode())

    def _tensor_ok(self, t: torch.Tensor, dtype, what: str):
        if not (t.is_cuda and t.is_contiguous() and t.dtype == dtype and t.device.index == self.device):
            raise W4a16Error(f"{what}: need a contiguous {dtype} CUDA tensor on device {self.device}")

    def set_tuning(self, key: str, value: int):
        self._ck(self._L.w4a16_set_tuning(self._h, key.encode(), int(value)))

    def launch_count(self) -> int:
        return int(self._L.w4a16_launch_count(self._h))

    def last_kernel(self) -> str:
        """Kernel instantiation launched by the last forward call."""
        return self._L.w4a16_last_kernel(self._h).decode()

    def weights_bytes(self) -> int:
        return int(self._L.w4a16_weights_bytes(self._h))

    def sync(self):
        self._ck(self._L.w4a16_sync(self._h))

    def debug_timeline(self, slots: int = 64 * 384 * 16) -> np.ndarray:
        out = np.zeros(slots, np.int64)
        self._ck(self._L.w4a16_debug_timeline(self._h, out.ctypes.data, slots))
        return out

    def kernel_status(self):
        """Raises if a kernel gave up on a bounded wait since the last check."""
        self._ck(self._L.w4a16_kernel_status(self._h))

    # -- weights ----------------------------------------------------------------------------
    def upload_lin(self, name: str, q: np.ndarray, s: np.ndarray, n: int, k: int):
        """upload.rs:4-13 -- g128 / f16-scale shorthand."""
        self.upload_lin_g(name, q, s, n, k, 128, False)

    def upload_lin_g(self, name: str, q, s, n: int, k: int, group: int, scale_bf16: bool = False):
        """upload.rs:15-65.  q: host bytes of u32 [n,k/8]; s: host bytes of 16-bit scales [n,k/group]."""
        qb = np.ascontiguousarray(q).view(np.uint8).ravel()
        sb = np.ascontiguousarray(s).view(np.uint8).ravel()
        self._ck(self._L.w4a16_upload_lin_g(self._h, name.encode(), qb.ctypes.data, qb.size, sb.ctypes.data,
                                            sb.size, n, k, group, int(scale_bf16)))

    def upload_lin_g_stream(self, name: str, n: int, k: int, group: int, scale_bf16: bool, fill):
        """upload.rs:1643 -- `fill(which, off, buf)` writes bytes [off, off+len(buf)) of q (which 0) or s (which 1)
        into the writable buffer it is given (a view of the decoder's pinned chunk)."""
        def tramp(_user, which, off, dst, length):
            buf = (C.c_ubyte * length).from_address(dst)
            fill(int(which), int(off), memoryview(buf).cast("B"))
        cb = _lib.FILL_FN(tramp)
        self._ck(self._L.w4a16_upload_lin_g_stream(self._h, name.encode(), n, k, group, int(scale_bf16), cb, None))

    def upload_lin_st(self, name: str, st: "SafeTensors", base: str):
        """gpu_engine/upload.rs:264-305: one linear of a mapped checkpoint, streamed to the device."""
        self._ck(self._L.w4a16_upload_lin_st(self._h, name.encode(), st._h, base.encode()))

    def save_lin_cache(self, name: str, path: str, source_tag: int):
        self._ck(self._L.w4a16_save_lin_cache(self._h, name.encode(), path.encode(), C.c_uint64(source_tag)))

    def load_lin_cache(self, name: str, path: str, source_tag: int):
        """Puts a linear back from its tile cache file with plain copies (no repack); raises on a stale file."""
        self._ck(self._L.w4a16_load_lin_cache(self._h, name.encode(), path.encode(), C.c_uint64(source_tag)))

    def upload_lin_g_dev(self, name: str, q: torch.Tensor, s: torch.Tensor, n: int, k: int, group: int,
                         scale_bf16: bool = False):
        """Device-source upload: q int32 [n,k/8], s int16/float16 [n,k/group] CUDA tensors."""
        if q.numel() * q.element_size() != n * (k // 2) or s.numel() * s.element_size() != n * (k // group) * 2:
            raise W4a16Error(f"upload_lin_g_dev {name}: tensor sizes do not match n={n} k={k} g{group}")
        if not (q.is_cuda and s.is_cuda and q.is_contiguous() and s.is_contiguous()):
            raise W4a16Error("upload_lin_g_dev: need contiguous CUDA tensors")
        self._ck(self._L.w4a16_upload_lin_g_dev(self._h, name.encode(), q.data_ptr(), s.data_ptr(), n, k, group,
                                                int(scale_bf16)))

    def lin_spec(self, name: str):
        n, k, g = C.c_int(), C.c_int(), C.c_int()
        self._ck(self._L.w4a16_lin_spec(self._h, name.encode(), C.byref(n), C.byref(k), C.byref(g)))
        return n.value, k.value, g.value

    def drop_lin(self, name: str):
        self._ck(self._L.w4a16_drop_lin(self._h, name.encode()))

    def unpack_lin(self, name: str):
        """Boundary-format (q int32 [n,k/8], s float16 [n,k/group]) rebuilt from the resident tiles."""
        n, k, g = self.lin_spec(name)
        q = torch.empty((n, k // 8), dtype=torch.int32, device=f"cuda:{self.device}")
        s = torch.empty((n, k // g), dtype=torch.float16, device=f"cuda:{self.device}")
        self._ck(self._L.w4a16_unpack_lin(self._h, name.encode(), q.data_ptr(), s.data_ptr(), _cur_stream()))
        return q, s

    def dequant_lin(self, name: str, f16: bool = False) -> torch.Tensor:
        n, k, _ = self.lin_spec(name)
        out = torch.empty((n, k), dtype=torch.float16 if f16 else torch.float32, device=f"cuda:{self.device}")
        self._ck(self._L.w4a16_dequant_lin(self._h, name.encode(), out.data_ptr(), OUT_F16 if f16 else OUT_F32,
                                           _cur_stream()))
        return out

    # -- forward ----------------------------------------------------------------------------
    def _out(self, t: int, n: int, f16: bool, dst):
        dt = torch.float16 if f16 else torch.float32
        if dst is None:
            return torch.empty((t, n), dtype=dt, device=f"cuda:{self.device}")
        self._tensor_ok(dst, dt, "dst")
        if dst.numel() != t * n:
            raise W4a16Error(f"dst has {dst.numel()} elements, need {t}x{n}")
        return dst

    def lin_forward(self, name: str, x16: torch.Tensor, t: int, dst: torch.Tensor | None = None,
                    out_f16: bool = False) -> torch.Tensor:
        """kernels/mod.rs:121-144: dst[t,n] = x16[t,k] @ W^T; GEMV for t<=8, tensor-core GEMM above."""
        n, k, _ = self.lin_spec(name)
        self._tensor_ok(x16, torch.float16, "x16")
        if x16.numel() != t * k:
            raise W4a16Error(f"lin_forward {name}: x has {x16.numel()} elements, need {t}x{k}")
        dst = self._out(t, n, out_f16, dst)
        self._ck(self._L.w4a16_lin_forward(self._h, name.encode(), x16.data_ptr(), dst.data_ptr(), t,
                                           OUT_F16 if out_f16 else OUT_F32, _cur_stream()))
        return dst

    def lin_forward_x32(self, name: str, x32: torch.Tensor, t: int, dst: torch.Tensor | None = None,
                        out_f16: bool = False) -> torch.Tensor:
        """lin_forward on f32 activations (kernels/gemv.rs:4-38 takes x as f32 holding f16 values)."""
        n, k, _ = self.lin_spec(name)
        self._tensor_ok(x32, torch.float32, "x32")
        if x32.numel() != t * k:
            raise W4a16Error(f"lin_forward_x32 {name}: x has {x32.numel()} elements, need {t}x{k}")
        dst = self._out(t, n, out_f16, dst)
        self._ck(self._L.w4a16_lin_forward_x32(self._h, name.encode(), x32.data_ptr(), dst.data_ptr(), t,
                                               OUT_F16 if out_f16 else OUT_F32, _cur_stream()))
        return dst

    def lin_forward_lane(self, name: str, x16: torch.Tensor, t: int) -> torch.Tensor:
        """The parity-gate kernel (gptq4.cu:825-951): f32 [t,n] in the CPU lane order, bit-identical to lane.rs."""
        n, k, _ = self.lin_spec(name)
        self._tensor_ok(x16, torch.float16, "x16")
        if x16.numel() != t * k:
            raise W4a16Error(f"lin_forward_lane {name}: x has {x16.numel()} elements, need {t}x{k}")
        dst = self._out(t, n, False, None)
        self._ck(self._L.w4a16_lin_forward_lane(self._h, name.encode(), x16.data_ptr(), dst.data_ptr(), t, _cur_stream()))
        return dst

    # -- int8 lm-head ------------------------------------------------------------------------
    def upload_head(self, w_bf16: np.ndarray, n: int, k: int):
        """upload.rs:1472-1569: bf16 [n,k] host matrix (uint16 bit patterns) -> int8 rows + f32 scales on the device."""
        w = np.ascontiguousarray(w_bf16, dtype=np.uint16)
        self._ck(self._L.w4a16_upload_head(self._h, w.ctypes.data, w.nbytes, n, k))

    def head_spec(self):
        n, k = C.c_int(0), C.c_int(0)
        self._ck(self._L.w4a16_head_spec(self._h, C.byref(n), C.byref(k)))
        return n.value, k.value

    def head_unpack(self):
        """The quantised lm-head as (int8 [n,k], f32 [n]) host arrays."""
        n, k = self.head_spec()
        q = np.zeros((n, k), np.int8)
        sc = np.zeros(n, np.float32)
        self._ck(self._L.w4a16_head_unpack(self._h, q.ctypes.data, sc.ctypes.data))
        return q, sc

    def head_forward(self, x32: torch.Tensor, t: int = 1, out: torch.Tensor | None = None) -> torch.Tensor:
        """kernels/gemv.rs:64-110 (head_gemv_launch / head_gemv_t_launch): f32 [t,k] -> f32 logits [t,n]."""
        n, k = self.head_spec()
        self._tensor_ok(x32, torch.float32, "x32")
        if x32.numel() != t * k:
            raise W4a16Error(f"head_forward: x has {x32.numel()} elements, need {t}x{k}")
        out = self._out(t, n, False, out)
        self._ck(self._L.w4a16_head_forward(self._h, x32.data_ptr(), out.data_ptr(), t, _cur_stream()))
        return out

    def sk_single_dev(self, name: str, x16: torch.Tensor, out: torch.Tensor | None = None, t: int = 1,
                      out_f16: bool = False) -> torch.Tensor:
        """kernels/decode.rs:89-127: split-K decode GEMV on one linear."""
        n, k, _ = self.lin_spec(name)
        self._tensor_ok(x16, torch.float16, "x16")
        if x16.numel() != t * k:
            raise W4a16Error(f"sk_single_dev {name}: x has {x16.numel()} elements, need {t}x{k}")
        out = self._out(t, n, out_f16, out)
        self._ck(self._L.w4a16_sk_single_dev(self._h, name.encode(), x16.data_ptr(), out.data_ptr(), t,
                                             OUT_F16 if out_f16 else OUT_F32, _cur_stream()))
        return out

    def sk_single_static(self, name: str, x16: torch.Tensor, out: torch.Tensor | None = None, t: int = 1,
                         out_f16: bool = False) -> torch.Tensor:
        """Same GEMV as :meth:`sk_single_dev`, for hosts that may not allocate device memory: the split-K
        scratch is a fixed 8 MiB array inside the library, shared by all calls (calls that overlap on the
        GPU race on it).  Shapes that need more are rejected.  Pass ``out``: this wrapper allocates the
        output tensor only when it is omitted.  Make the first call on a device outside stream capture."""
        n, k, _ = self.lin_spec(name)
        self._tensor_ok(x16, torch.float16, "x16")
        if x16.numel() != t * k:
            raise W4a16Error(f"sk_single_static {name}: x has {x16.numel()} elements, need {t}x{k}")
        out = self._out(t, n, out_f16, out)
        self._ck(self._L.w4a16_sk_single_static(self._h, name.encode(), x16.data_ptr(), out.data_ptr(), t,
                                                OUT_F16 if out_f16 else OUT_F32, _cur_stream()))
        return out

    # -- row-parallel tensor parallelism ---------------------------------------------------------
    def tp_setup(self, rank: int, world: int, max_rows: int, group=None):
        """Creates this rank's exchange block and maps the peers' (handles travel over torch.distributed)."""
        import torch.distributed as dist
        mine = C.create_string_buffer(64)
        self._ck(self._L.w4a16_tp_create(self._h, rank, world, max_rows, mine))
        handles = [None] * world
        dist.all_gather_object(handles, bytes(mine.raw), group=group)
        blob = C.create_string_buffer(b"".join(handles), 64 * world)
        self._ck(self._L.w4a16_tp_connect(self._h, blob))
        dist.barrier(group=group)

    def tp_rearm(self):
        """Resets this rank's exchange block after an abandoned fused all-reduce; every rank calls it between
        two host barriers."""
        self._ck(self._L.w4a16_tp_rearm(self._h))

    def sk_single_allreduce(self, name: str, x16: torch.Tensor, out: torch.Tensor | None = None, t: int = 1,
                            out_f16: bool = False) -> torch.Tensor:
        """Row-parallel GEMV whose kernel also sums the partial outputs over the ranks (peer stores)."""
        n, k, _ = self.lin_spec(name)
        self._tensor_ok(x16, torch.float16, "x16")
        if x16.numel() != t * k:
            raise W4a16Error(f"sk_single_allreduce {name}: x has {x16.numel()} elements, need {t}x{k}")
        out = self._out(t, n, out_f16, out)
        self._ck(self._L.w4a16_sk_single_allreduce(self._h, name.encode(), x16.data_ptr(), out.data_ptr(), t,
                                                   OUT_F16 if out_f16 else OUT_F32, _cur_stream()))
        return out

    def sk_multi_dev(self, names, x16: torch.Tensor, outs=None, t: int = 1, out_f16: bool = False):
        """kernels/decode.rs:23-57: q|k|v or gate|up in one launch (same x, same k)."""
        specs = [self.lin_spec(nm) for nm in names]
        self._tensor_ok(x16, torch.float16, "x16")
        if x16.numel() != t * specs[0][1]:
            raise W4a16Error("sk_multi_dev: x size does not match t*k")
        if outs is None:
            outs = [None] * len(names)
        outs = [self._out(t, sp[0], out_f16, o) for sp, o in zip(specs, outs)]
        arr_n = (C.c_char_p * len(names))(*[nm.encode() for nm in names])
        arr_o = (C.c_void_p * len(names))(*[o.data_ptr() for o in outs])
        self._ck(self._L.w4a16_sk_multi_dev(self._h, arr_n, len(names), x16.data_ptr(), arr_o, t,
                                            OUT_F16 if out_f16 else OUT_F32, _cur_stream()))
        return outs

    def lin_forward_host(self, name: str, x16: np.ndarray, t: int, out_f16: bool = False,
                         out: np.ndarray | None = None) -> np.ndarray:
        """Host-buffer forward: H2D of x, the linear, D2H of the result, synchronised."""
        n, k, _ = self.lin_spec(name)
        xb = np.ascontiguousarray(x16).view(np.uint16).ravel()
        if xb.size != t * k:
            raise W4a16Error(f"lin_forward_host {name}: x has {xb.size} elements, need {t}x{k}")
        if out is None:
            out = np.empty((t, n), np.float16 if out_f16 else np.float32)
        self._ck(self._L.w4a16_lin_forward_host(self._h, name.encode(), xb.ctypes.data, out.ctypes.data, t,
                                                OUT_F16 if out_f16 else OUT_F32))
        return out

    # -- graphs (ctx/graph.rs:4-85) -----------------------------------------------------------
    def stream_ptr(self) -> int:
        return int(self._L.w4a16_stream(self._h))

    def capture_begin(self):
        self._ck(self._L.w4a16_capture_begin(self._h))

    def capture_end(self) -> int:
        g = C.c_void_p()
        self._ck(self._L.w4a16_capture_end(self._h, C.byref(g)))
        return g.value

    def graph_launch(self, g: int):
        self._ck(self._L.w4a16_graph_launch(self._h, C.c_void_p(g)))

    def graph_destroy(self, g: int):
        self._ck(self._L.w4a16_graph_destroy(self._h, C.c_void_p(g)))

    def graph_step_host(self, g: int, x_host: torch.Tensor, x_dev: torch.Tensor, y_dev: torch.Tensor,
                        y_host: torch.Tensor):
        """graphs.rs:202 shape: H2D of the step input, graph replay, D2H of the result, sync."""
        self._ck(self._L.w4a16_graph_step_host(
            self._h, C.c_void_p(g), x_host.data_ptr(), x_dev.data_ptr(), x_host.numel() * x_host.element_size(),
            y_dev.data_ptr(), y_host.data_ptr(), y_host.numel() * y_host.element_size()))

    # -- MoE (upload.rs:795-812,1021-1235; moe/mod.rs:263-447) --------------------------------------
    def set_moe(self, n_experts: int, top_k: int, moe_ffn: int, hidden: int, group: int = 32,
                expert_first: int = 0, expert_count: int | None = None):
        cnt = n_experts - expert_first if expert_count is None else expert_count
        self._ck(self._L.w4a16_set_moe(self._h, n_experts, top_k, moe_ffn, hidden, group, expert_first, cnt))
        self._moe = (n_experts, top_k, moe_ffn, hidden, group, expert_first, cnt)

    def upload_experts(self, layer: int, w13_q, w13_s, w2_q, w2_s, scale_bf16: bool = False):
        """Local experts of one layer from host arrays (expert-major, gate rows then up rows in w13)."""
        if isinstance(w13_q, torch.Tensor):
            self._ck(self._L.w4a16_upload_experts_dev(self._h, layer, w13_q.data_ptr(), w13_s.data_ptr(),
                                                      w2_q.data_ptr(), w2_s.data_ptr(), int(scale_bf16)))
            return
        ne, k, f, h, g, _, cnt = self._moe
        arrs = [np.ascontiguousarray(a) for a in (w13_q, w13_s, w2_q, w2_s)]
        want = [cnt * 2 * f * h // 2, cnt * 2 * f * (h // g) * 2, cnt * h * f // 2, cnt * h * (f // g) * 2]
        for a, w in zip(arrs, want):
            if a.nbytes != w:
                raise W4a16Error(f"upload_experts: array of {a.nbytes} bytes, expected {w}")
        self._ck(self._L.w4a16_upload_experts(self._h, layer, *[a.ctypes.data for a in arrs], int(scale_bf16)))

    def moe_topk(self, logits: torch.Tensor):
        """moe.cu:686-759 / mod.rs:168-185: (idx int32 [t,k], wt float32 [t,k])."""
        ne, k = self._moe[0], self._moe[1]
        self._tensor_ok(logits, torch.float32, "logits")
        t = logits.numel() // ne
        idx = torch.empty((t, k), dtype=torch.int32, device=logits.device)
        wt = torch.empty((t, k), dtype=torch.float32, device=logits.device)
        self._ck(self._L.w4a16_moe_topk(self._h, logits.data_ptr(), idx.data_ptr(), wt.data_ptr(), t, _cur_stream()))
        return idx, wt

    def moe_ffn_dev_t(self, il: int, logits: torch.Tensor, x16: torch.Tensor, t: int,
                      out: torch.Tensor | None = None, out_f16: bool = False) -> torch.Tensor:
        """moe/mod.rs:263: y[t,h] over the local experts (sum y over ranks under expert parallelism)."""
        ne, k, f, h, g, _, _ = self._moe
        self._tensor_ok(logits, torch.float32, "logits")
        self._tensor_ok(x16, torch.float16, "x16")
        if logits.numel() != t * ne or x16.numel() != t * h:
            raise W4a16Error("moe_ffn_dev_t: logits/x sizes do not match t")
        out = self._out(t, h, out_f16, out)
        self._ck(self._L.w4a16_moe_ffn(self._h, il, logits.data_ptr(), x16.data_ptr(), out.data_ptr(), t,
                                       OUT_F16 if out_f16 else OUT_F32, _cur_stream()))
        return out


class SafeTensors:
    """crates/core/src/st.rs StArchive + the linear scan of crates/core/src/w4a16.rs:108-191, over the C ABI
    (host only: needs no device)."""

    def __init__(self, path: str):
        self._L = _lib.lib()
        h = C.c_void_p()
        if self._L.w4a16_st_open(str(path).encode(), C.byref(h)) != 0:
            raise W4a16Error(self._L.w4a16_st_error().decode())
        self._h = h

    def close(self):
        if getattr(self, "_h", None):
            self._L.w4a16_st_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def linears(self):
        """[(base, n, k, group, scale_bf16)] in name order."""
        out = []
        buf = C.create_string_buffer(512)
        n, k, g, b = C.c_int(), C.c_int(), C.c_int(), C.c_int()
        for i in range(self._L.w4a16_st_lin_count(self._h)):
            if self._L.w4a16_st_lin_at(self._h, i, buf, 512, C.byref(n), C.byref(k), C.byref(g), C.byref(b)) != 0:
                raise W4a16Error(self._L.w4a16_st_error().decode())
            out.append((buf.value.decode(), n.value, k.value, g.value, bool(b.value)))
        return out

    def tag(self, base: str) -> int:
        t = C.c_uint64()
        if self._L.w4a16_st_lin_tag(self._h, base.encode(), C.byref(t)) != 0:
            raise W4a16Error(self._L.w4a16_st_error().decode())
        return int(t.value)
