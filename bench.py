#!/usr/bin/env python
"""Headline benchmark of the W4A16 matmul path on B200.

Workload (N=1): one decode token (M=1) through the W4A16 linears of a 64-layer 27B-class dense
decoder -- per layer qkv (K=5120,N=7168), o_proj (6144,5120), gate_up (5120,34816) and down
(17408,5120); int4 sym g128 weights, f16 scales and activations -- i.e. the decode-GEMV shapes
of the baseline's single-GPU sweep laid out as the 64-layer stack, 11.07 GB of weights per step, so
every launch streams from HBM (the stack is ~88x the L2).  A step is replayed as one CUDA graph of
256 GEMV launches, the way the reference replays its decode chain.

  value     whole-job GB/s = algorithmic bytes of the step / device time (inputs resident in HBM);
            the timed region of `--steps` steps is repeated and the median repeat is reported
  e2e       same metric through the host-buffer step call: H2D of the token's activations from pinned
            memory + graph replay + D2H of the result + sync, every step (wall clock)
  roofline  the GEMV kernel against the measured HBM copy bandwidth (per GPU)
  roofline_prefill  the tensor-core GEMM at M=4096 against the measured and nominal f16 dense rates
  cpu_baseline  the CPU oracle (restatement of the reference quant lane) timed on this host

With --gpus N>1 (torchrun) the same stack is tensor-parallel: qkv/gate_up column-parallel, o_proj/down
row-parallel with the all-reduce fused into the GEMV; total work is fixed ("strong" scaling).  The N>1 line
also carries a parity block (outputs of the LAST timed replay against the CPU oracle), a prefill layer with
the row-parallel all-reduce overlapped, and the expert-parallel MoE layer at T = 1, 64, 4096.
`--impl reference` times the reference's CPU algorithm for the same workload on the host cores.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from llm170_b200 import synth  # noqa: E402

LAYER_ORDER = ["qkv", "o_proj", "gate_up", "down"]
METRIC = "W4A16 decode GEMV HBM GB/s (M=1), 27B-class 64-layer linear stack"
WORKLOAD = ("decode M=1, 27B-class dense linear stack (qkv 5120x7168, o_proj 6144x5120, gate_up 5120x34816, "
            "down 17408x5120), int4 sym g128, f16 scales")
REPEATS = 5   # timed regions per measurement; the median is reported


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p)), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples SM clocks / throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self, settle_s: float = 0.5):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
            time.sleep(settle_s)   # nvidia-smi needs a few hundred ms before its first sample
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [c.strip() for c in line.split(",")]))

    def stop(self, t_begin: float, t_end: float):
        """Summary of the samples taken between t_begin and t_end (perf_counter), all samples if none fell inside."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        time.sleep(0.1)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

        def summarise(rows):
            sm, mx, reasons = [], [], set()
            for _, r in rows:
                if len(r) < 6:
                    continue
                try:
                    sm.append(float(r[0]))
                    mx.append(float(r[1]))
                except ValueError:
                    continue
                for nm, v in zip(names, r[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(nm)
            return sm, mx, reasons

        inside = [(t, r) for t, r in self.rows if t_begin - 0.05 <= t <= t_end + 0.05]
        sm, mx, reasons = summarise(inside if inside else self.rows)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "samples_inside_timed_region": len(inside)}


def layer_shapes(world: int):
    """(K, N, kind) per rank for tensor-parallel degree `world` (world=1: the full layer)."""
    out = {}
    for nm, (k, n) in synth.DENSE_27B.items():
        if nm in ("qkv", "gate_up"):
            out[nm] = (k, n // world, "col")
        else:
            out[nm] = (k // world, n, "row")
    return out


def step_bytes(m: int = 1) -> int:
    """Algorithmic bytes of ONE layer (its four linears) at m tokens."""
    return sum(synth.decode_bytes(n, k, m) for (k, n) in synth.DENSE_27B.values())


# ------------------------------------------------------------------------------------------------
def run_reference_arm(args, rank: int):
    """The reference's CPU algorithm (oracle restatement of crates/core/src/quant/lane.rs) on all host threads.
    A step is a bounded sample of the workload: `sample_layers` whole layers (all four linears, all rows) at M=1;
    `ms_per_step` is the measured wall time of that sample, `value` the bytes it covers over that time."""
    if rank != 0:
        return
    import oracle
    oracle.build()
    cores = os.cpu_count() or 1
    sample_layers = 2
    lins = {}
    for li in range(sample_layers):
        for nm, (k, n) in synth.DENSE_27B.items():
            lins[(li, nm)] = synth.make_linear(n, k, 128, seed=4000 + li * 10 + len(nm)) + (k, n)
    xs = {k: synth.make_acts(1, k, seed=k) for k in (5120, 6144, 17408)}

    def one_step():
        t0 = time.perf_counter()
        for li in range(sample_layers):
            for nm in LAYER_ORDER:
                q, s, k, n = lins[(li, nm)]
                oracle.linear_lane(q, s, xs[k], 1, n, k, 128, nthreads=cores)
        return time.perf_counter() - t0

    for _ in range(args.warmup):
        one_step()
    tot = sum(one_step() for _ in range(args.steps))
    s_per_step = tot / args.steps
    gbs = step_bytes() * sample_layers / s_per_step / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": s_per_step * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16 x int4 -> f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "layers": 64, "l2": "inputs larger than cache"},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": f"{sample_layers} of 64 layers per step (all four linears, all rows, M=1)",
                         "ms_per_64_layer_step_scaled": s_per_step * 1e3 * 64 / sample_layers},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
def upload_synthetic_head(dec, n, k, device):
    """A seeded N(0, 0.02) lm-head as bf16 bit patterns, made on the device and passed through the host boundary."""
    import torch
    gen = torch.Generator(device=device)
    gen.manual_seed(77)
    w = (torch.randn((n, k), generator=gen, device=device, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    dec.upload_head(w.view(torch.int16).cpu().numpy().view(np.uint16), n, k)


def lm_head(dec, device, st, peaks, g):
    """The int8 lm-head GEMV (vocabulary x hidden int8 bytes per token: the largest weight stream of a decode step
    after the layers) at t = 1 and 8, with a parity check of 64 rows against the oracle's lane-order sum."""
    import torch
    n, k = synth.LM_HEAD_27B
    upload_synthetic_head(dec, n, k, device)
    out = {"vocab": n, "hidden": k, "kernel": None}
    with torch.cuda.stream(st):
        for t in (1, 8):
            gen = torch.Generator(device=device)
            gen.manual_seed(5 + t)
            x = torch.randn((t, k), generator=gen, device=device, dtype=torch.float32)
            y = torch.empty((t, n), device=device, dtype=torch.float32)
            dec.head_forward(x, t, out=y)
            st.synchronize()
            ts = []
            for _ in range(5):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(st)
                dec.head_forward(x, t, out=y)
                e1.record(st)
                e1.synchronize()
                ts.append(e0.elapsed_time(e1) * 1e-3)
            sec = float(np.median(ts))
            nbytes = n * k + n * 4 + t * k * 4 + t * n * 4
            out[f"t{t}"] = {"us": sec * 1e6, "GB/s": nbytes / sec / 1e9, "frac_of_hbm": nbytes / sec / 1e9 / peaks["hbm_gbs"]}
            if t == 1:
                import oracle
                q, sc = dec.head_unpack()
                rows = np.linspace(0, n - 1, 64).astype(np.int64)
                xs = x.cpu().numpy()
                expect = oracle.head_gemv_i8(q[rows], sc[rows], xs, 1)[0]
                bound = 1e-5 * (np.abs(xs[0]).astype(np.float64) @ np.abs(q[rows]).astype(np.float64).T) * sc[rows]
                err = np.abs(y[0].cpu().numpy()[rows].astype(np.float64) - expect)
                out["parity_64_rows"] = {"ok": bool((err <= bound).all()), "max_err_over_bound": float((err / bound).max())}
    out["kernel"] = dec.last_kernel()
    return out


def run_case(args, dec, device):
    """ONE small case instead of the benchmark (what the profiler captures in profiles/ run)."""
    import torch
    if args.case.startswith("head:"):
        T = int(args.case.split(":")[1])
        n, k = synth.LM_HEAD_27B
        upload_synthetic_head(dec, n, k, device)
        gen = torch.Generator(device=device)
        gen.manual_seed(1)
        xh = torch.randn((T, k), generator=gen, device=device, dtype=torch.float32)
        yh = torch.empty((T, n), device=device, dtype=torch.float32)
        fn = lambda: dec.head_forward(xh, T, out=yh)  # noqa: E731
    elif args.case.startswith("moe:"):
        T = int(args.case.split(":")[1])
        mo = synth.MOE_35B
        ne, h, f, kk, grp = mo["n_experts"], mo["hidden"], mo["moe_ffn"], mo["top_k"], mo["group"]
        dec.set_moe(ne, kk, f, h, grp)
        q13, s13 = synth.make_linear_cuda(ne * 2 * f, h, grp, seed=900, device=device)
        q2, s2 = synth.make_linear_cuda(ne * h, f, grp, seed=950, device=device)
        dec.upload_experts(0, q13, s13, q2, s2)
        gen = torch.Generator(device=device)
        gen.manual_seed(3)
        lg = torch.randn((T, ne), generator=gen, device=device, dtype=torch.float32)
        xm = torch.randn((T, h), generator=gen, device=device, dtype=torch.float32).to(torch.float16)
        ym = torch.empty((T, h), device=device, dtype=torch.float32)
        fn = lambda: dec.moe_ffn_dev_t(0, lg, xm, T, out=ym)  # noqa: E731
    else:
        kind, nm, m = args.case.split(":")
        m = int(m)
        k, n = synth.DENSE_27B[nm]
        q, s = synth.make_linear_cuda(n, k, 128, seed=7, device=device)
        dec.upload_lin_g_dev("case", q, s, n, k, 128)
        gen = torch.Generator(device=device)
        gen.manual_seed(1)
        xg = (torch.randn((m, k), generator=gen, device=device) / (k ** 0.5 if kind == "gemm" else 1.0)).to(torch.float16)
        yg = torch.empty((m, n), device=device, dtype=torch.float16)
        fn = (lambda: dec.lin_forward("case", xg, m, dst=yg, out_f16=True)) if kind == "gemm" else \
             (lambda: dec.sk_single_dev("case", xg, out=yg, t=m, out_f16=True))
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        fn()
    e1.record()
    e1.synchronize()
    dec.kernel_status()
    print(json.dumps({"case": args.case, "launches": args.steps + 1, "kernel": dec.last_kernel(),
                      "us_per_call": e0.elapsed_time(e1) * 1e3 / args.steps}))


def run_b200_arm(args, rank: int, world: int, local_rank: int):
    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the W4A16 path has no CPU fallback "
                         "(use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    # the timed binary is built from the checked-out sources (a no-op when the recorded source hash matches)
    from llm170_b200 import build as lib_build
    if local_rank == 0:
        lib_build.build()
    if world > 1:
        dist.barrier()
    from llm170_b200.w4a16_dec import W4a16Dec
    peaks, peak_kind = load_peaks()

    dec = W4a16Dec(local_rank)
    try:
        for kv in args.tune:
            key, val = kv.split("=")
            dec.set_tuning(key, int(val))
        if args.case:
            run_case(args, dec, device)
            return
        line = measure(args, dec, device, rank, world, local_rank, peaks, peak_kind)
        if rank == 0:
            print(json.dumps(line), flush=True)
    finally:
        # every tensor made on the decoder's stream is gone by now (they were locals of measure()); give torch's
        # caching allocator its blocks back before the stream goes away, then leave through a normal return
        gc.collect()
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        dec.close()
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()


def measure(args, dec, device, rank, world, local_rank, peaks, peak_kind):
    import torch
    import torch.distributed as dist

    L = args.layers
    shapes = layer_shapes(world)
    t_build = time.time()
    for li in range(L):
        for nm in LAYER_ORDER:
            k, n, kind = shapes[nm]
            # each rank generates only its own shard (seeded per layer, linear and rank)
            q, s = synth.make_linear_cuda(n, k, 128, seed=4_000_000 + li * 1000 + LAYER_ORDER.index(nm) * 16 + rank,
                                          device=device)
            dec.upload_lin_g_dev(f"l{li}.{nm}", q, s, n, k, 128)
            del q, s
    torch.cuda.synchronize()
    t_build = time.time() - t_build

    # activations: fixed device buffers, one per linear (values N(0,1) f16; the same on every rank)
    g = torch.Generator(device=device)
    g.manual_seed(1)
    xb = {nm: torch.randn((8, shapes[nm][0]), generator=g, device=device, dtype=torch.float32).to(torch.float16)
          for nm in LAYER_ORDER}
    yb = {nm: torch.empty((8, shapes[nm][1]), device=device, dtype=torch.float16) for nm in LAYER_ORDER}
    x_host = torch.empty((1, shapes["qkv"][0]), dtype=torch.float16).pin_memory()
    x_host.copy_(xb["qkv"][:1].cpu())
    y_host = torch.empty((1, shapes["down"][1]), dtype=torch.float16).pin_memory()

    st = torch.cuda.ExternalStream(dec.stream_ptr(), device=device)

    if world > 1:
        dec.tp_setup(rank, world, max_rows=max(shapes[nm][1] for nm in LAYER_ORDER if shapes[nm][2] == "row"))

    kernels_seen = {}
    kernel_bytes = {}      # weight bytes each kernel streams: the dominant kernel is the one that streams most

    def launch_lin(li, nm, m):
        if world > 1 and shapes[nm][2] == "row":
            # row-parallel: the GEMV kernel itself sums the partial outputs over the ranks (peer stores)
            dec.sk_single_allreduce(f"l{li}.{nm}", xb[nm][:m], out=yb[nm][:m], t=m, out_f16=True)
        else:
            dec.sk_single_dev(f"l{li}.{nm}", xb[nm][:m], out=yb[nm][:m], t=m, out_f16=True)
        kernels_seen[dec.last_kernel()] = kernels_seen.get(dec.last_kernel(), 0) + 1
        kernel_bytes[dec.last_kernel()] = kernel_bytes.get(dec.last_kernel(), 0) + shapes[nm][0] * shapes[nm][1] // 2

    def enqueue_step(m: int):
        for li in range(L):
            for nm in LAYER_ORDER:
                launch_lin(li, nm, m)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def capture(fn):
        """Warm scratch, then capture fn() on the decoder stream; returns (graph, launches)."""
        with torch.cuda.stream(st):
            fn()
            st.synchronize()
            if world > 1:
                dist.barrier()                    # every rank replays the same sequence of exchanges
            c0 = dec.launch_count()
            dec.capture_begin()
            fn()
            return dec.capture_end(), dec.launch_count() - c0

    def time_graph(gx, n_launch: int) -> float:
        """Device time (ms) of n_launch replays on the decoder stream, max over ranks."""
        with torch.cuda.stream(st):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(st)
            for _ in range(n_launch):
                dec.graph_launch(gx)
            e1.record(st)
            e1.synchronize()
            ms = e0.elapsed_time(e1)
        if world > 1:
            tms = torch.tensor([ms], device=device)
            dist.all_reduce(tms, op=dist.ReduceOp.MAX)
            ms = float(tms.item())
        return ms

    kernels_seen.clear()
    gx1, launches_per_step = capture(lambda: enqueue_step(1))
    step_kernels = {k: v // 2 for k, v in kernels_seen.items()}     # counted once warm, once captured
    time_graph(gx1, args.warmup)

    # ---- the timed region: exactly `steps` steps between barriers, REPEATS times; the median repeat is the value
    sampler = ClockSampler(local_rank)
    sampler.start()
    rep_ms = []
    t_begin = time.perf_counter()
    for _ in range(REPEATS):
        barrier()
        rep_ms.append(time_graph(gx1, args.steps))
        barrier()
    t_end = time.perf_counter()
    clocks = sampler.stop(t_begin, t_end)
    ms = float(np.median(rep_ms))
    ms_per_step = ms / args.steps
    bytes_step = step_bytes(1) * L
    value = bytes_step / (ms_per_step * 1e-3) / 1e9

    # ---- parity of the LAST timed replay (N > 1): the outputs it left in yb against the CPU oracle ---------------
    parity = None
    if world > 1:
        parity = tp_parity_of_last_replay(dec, dist, device, rank, world, shapes, xb, yb, L)

    # ---- e2e: host buffers, H2D + graph + D2H + sync every step (wall clock, max over ranks) --------
    xdev, ydev = xb["qkv"][:1], yb["down"][:1]
    for _ in range(max(3, args.warmup)):
        dec.graph_step_host(gx1, x_host, xdev, ydev, y_host)
    e2e_reps = []
    for _ in range(REPEATS):
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            dec.graph_step_host(gx1, x_host, xdev, ydev, y_host)
        e2e_s = (time.perf_counter() - t0) / args.steps
        if world > 1:
            te = torch.tensor([e2e_s], device=device)
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
            e2e_s = float(te.item())
        e2e_reps.append(e2e_s)
    e2e_s = float(np.median(e2e_reps))
    e2e = {"value": bytes_step / e2e_s / 1e9, "unit": "GB/s", "ms_per_step": e2e_s * 1e3,
           "h2d_bytes_per_step": x_host.numel() * 2 * world, "d2h_bytes_per_step": y_host.numel() * 2 * world}
    dec.graph_destroy(gx1)

    extras = {}
    roofline_prefill = None
    if not args.no_extras:
        extras["per_launch_M1" if world == 1 else "tp_M1_per_launch"] = per_shape_sweep(
            dec, dist, device, st, world, shapes, xb, yb, L, peaks, capture, time_graph, ms_tokens=(1,) if world > 1 else (1, 2, 4, 8))
        if world == 1:
            roofline_prefill, extras["prefill"] = prefill_sweep(dec, device, st, shapes, L, peaks, g)
            extras["moe_35b_a3b_layer"] = moe_layer(dec, dist, device, st, rank, world, g)
            extras["lm_head_int8"] = lm_head(dec, device, st, peaks, g)
        else:
            extras["tp_prefill_M4096"] = tp_prefill(dec, dist, device, st, shapes, L, g)
            extras["ep_moe_35b_a3b_layer"] = moe_layer(dec, dist, device, st, rank, world, g)
        dec.kernel_status()

    # ---- CPU baseline (rank 0, N=1): the oracle on a bounded sample ----------------------------------
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        import oracle
        oracle.build()
        cores = os.cpu_count() or 1
        sample_layers = min(L, 24)      # about 25 core-seconds of the lane dot on 16 threads
        host = []
        for li in range(sample_layers):
            for nm in LAYER_ORDER:
                k, n, _ = shapes[nm]
                q, s = dec.unpack_lin(f"l{li}.{nm}")
                host.append((q.cpu().numpy().view(np.uint32), s.cpu().numpy().view(np.uint16),
                             xb[nm][:1].cpu().numpy().view(np.uint16), n, k, nm, li))
        t0 = time.perf_counter()
        maxerr = 0.0
        for q, s, x, n, k, nm, li in host:
            ref = oracle.linear_lane(q, s, x, 1, n, k, 128, nthreads=cores)
            if li == 0:  # parity spot check of the exact tensors that were timed on the GPU
                got = dec.sk_single_dev(f"l{li}.{nm}", xb[nm][:1], t=1).cpu().numpy()
                maxerr = max(maxerr, float(np.abs(got - ref).max()))
        cpu_s = time.perf_counter() - t0
        cpu_gbs = step_bytes(1) * sample_layers / cpu_s / 1e9
        cpu_baseline = {"value": cpu_gbs, "unit": "GB/s", "cores": cores, "kind": "port",
                        "sample": f"{sample_layers} of {L} layers (all four linears, all rows, M=1), "
                                  f"{cpu_s:.1f} s of wall time on {cores} threads ({cpu_s * cores:.0f} core-seconds)",
                        "max_abs_err_gpu_vs_cpu_layer0": maxerr}

    per_gpu = value / world   # every GPU streams 1/N of the bytes against its own HBM
    top_kernel = max(kernel_bytes, key=kernel_bytes.get) if kernel_bytes else dec.last_kernel()
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16 x int4 -> f32", "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "layers": L, "parallelism": f"tp{world}" if world > 1 else "single",
                   "l2": f"inputs larger than L2 ({bytes_step / 1e9:.2f} GB of weights per step)",
                   "launch": "cuda graph replay" + (", all-reduce fused into the row-parallel GEMV (peer stores)" if world > 1 else ""),
                   "repeats": REPEATS, "repeat_ms": [round(r, 4) for r in rep_ms], "build_s": round(t_build, 1)},
        "roofline": {"bound": "hbm", "kernel": top_kernel, "kernels_per_step": step_kernels,
                     "achieved": per_gpu, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": per_gpu / peaks["hbm_gbs"],
                     "per": "GPU", "peak_kind": peak_kind, "frac_of_nominal_8TBps": per_gpu / 8000.0,
                     # dram bytes per launch are not measured inside this run; the ncu capture of this kernel
                     # under profiles/ gives read+write traffic / algorithmic bytes = 1.002
                     "traffic": None,
                     "launches_per_step": launches_per_step,
                     "avg_launch_us": ms_per_step * 1e3 / launches_per_step,
                     "algorithmic_bytes_per_launch": bytes_step / launches_per_step / world},
        "e2e": e2e, "gpu_launches": launches_per_step * args.steps * REPEATS, "clocks": clocks,
        "cpu_baseline": cpu_baseline,
    }
    if roofline_prefill is not None:
        line["roofline_prefill"] = roofline_prefill
    if parity is not None:
        line["parity"] = parity
    line["extras"] = extras
    return line


def tp_parity_of_last_replay(dec, dist, device, rank, world, shapes, xb, yb, L):
    """The last layer's four linears as the last graph replay left them in yb, against the lane oracle on rank 0
    (shards gathered with all_gather; the timed outputs are f16, so the comparison allows their rounding)."""
    import torch
    out = {}
    li = L - 1
    worst = {"col": 0.0, "row": 0.0}
    for nm in LAYER_ORDER:
        k, n, kind = shapes[nm]
        q, s = dec.unpack_lin(f"l{li}.{nm}")
        qs = [torch.empty_like(q) for _ in range(world)]
        ss = [torch.empty_like(s) for _ in range(world)]
        xs = [torch.empty_like(xb[nm][:1]) for _ in range(world)]
        ys = [torch.empty_like(yb[nm][:1]) for _ in range(world)]
        dist.all_gather(qs, q)
        dist.all_gather(ss, s)
        dist.all_gather(xs, xb[nm][:1].contiguous())
        dist.all_gather(ys, yb[nm][:1].contiguous())
        if rank == 0:
            import oracle
            oracle.build()
            if kind == "col":
                qf, sf = torch.cat(qs, 0), torch.cat(ss, 0)
                xf, yf = xs[0], torch.cat(ys, 1)
                nf, kf = n * world, k
            else:
                qf, sf = torch.cat(qs, 1), torch.cat(ss, 1)
                xf, yf = torch.cat(xs, 1), ys[0]
                nf, kf = n, k * world
                for r in range(1, world):          # every rank holds the same all-reduced output
                    assert torch.equal(ys[r], ys[0]), f"rank {r} disagrees on {nm}"
            want = oracle.linear_lane(qf.cpu().numpy().view(np.uint32), sf.cpu().numpy().view(np.uint16),
                                      xf.cpu().numpy().view(np.uint16), 1, nf, kf, 128)
            got = yf.float().cpu().numpy()
            err = float(np.abs(got - want).max())
            # f16 output: half an ulp at |y| plus the 2e-3 gate on the f32 sums
            bound = float(np.abs(want).max()) * 2.0 ** -11 + 2e-3
            out[nm] = {"max_abs_err": err, "bound": bound, "ok": err <= bound}
            worst[kind] = max(worst[kind], err)
    # rank 0 has spent seconds in the oracle: the others wait here, so that the next fused launches of all ranks
    # start together (the in-kernel wait for the peers is bounded at about a second)
    dist.barrier()
    if rank == 0:
        return {"checked": f"layer {li} of the last timed graph replay, all rows, f16 outputs vs f32 lane oracle",
                "tp_col_max_abs_err": worst["col"], "tp_row_fused_allreduce_max_abs_err": worst["row"],
                "per_linear": out, "ok": all(v["ok"] for v in out.values())}
    return None


def per_shape_sweep(dec, dist, device, st, world, shapes, xb, yb, L, peaks, capture, time_graph, ms_tokens):
    """Per-shape launch time, each shape rotating over all layers (> L2), for the given token counts.
    fixed_cost_us = measured time minus the time the launch's algorithmic bytes take at the measured HBM rate."""
    import torch
    res = {}
    for m in ms_tokens:
        per = {}
        for nm in LAYER_ORDER:
            k, n, kind = shapes[nm]

            def shape_pass():
                for li in range(L):
                    if world > 1 and kind == "row":
                        dec.sk_single_allreduce(f"l{li}.{nm}", xb[nm][:m], out=yb[nm][:m], t=m, out_f16=True)
                    else:
                        dec.sk_single_dev(f"l{li}.{nm}", xb[nm][:m], out=yb[nm][:m], t=m, out_f16=True)
            gsh, _ = capture(shape_pass)
            time_graph(gsh, 3)
            reps = 5
            us = time_graph(gsh, reps) * 1e3 / (reps * L)
            dec.graph_destroy(gsh)
            b = synth.decode_bytes(n, k, m)
            per[nm] = {"us": round(us, 3), "GBps": round(b / us / 1e3, 1), "kernel": dec.last_kernel(),
                       "frac_measured_hbm": round(b / us / 1e3 / peaks["hbm_gbs"], 4),
                       "fixed_cost_us": round(us - b / peaks["hbm_gbs"] / 1e3, 3)}
            if world > 1:
                per[nm].update({"shard": [n, k], "kind": kind})
        res[f"M{m}"] = per
    return res if len(ms_tokens) > 1 else res[f"M{ms_tokens[0]}"]


def prefill_sweep(dec, device, st, shapes, L, peaks, g):
    """Tensor-core GEMM, TFLOP/s per shape, rotating over 8 layers; the M=4096 row is the roofline_prefill block."""
    import torch
    pre = {}
    with torch.cuda.stream(st):
        for m in (512, 1024, 4096):
            per = {}
            for nm in LAYER_ORDER:
                k, n, _ = shapes[nm]
                xg = (torch.randn((m, k), generator=g, device=device, dtype=torch.float32) / (k ** 0.5)).to(torch.float16)
                yg = torch.empty((m, n), device=device, dtype=torch.float16)
                nl = min(L, 8)
                for li in range(nl):
                    dec.lin_forward(f"l{li}.{nm}", xg, m, dst=yg, out_f16=True)
                st.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                reps = 3
                e0.record(st)
                for _ in range(reps):
                    for li in range(nl):
                        dec.lin_forward(f"l{li}.{nm}", xg, m, dst=yg, out_f16=True)
                e1.record(st)
                e1.synchronize()
                us = e0.elapsed_time(e1) * 1e3 / (reps * nl)
                tf = synth.gemm_flops(n, k, m) / us / 1e6
                per[nm] = {"us": round(us, 2), "TFLOPs": round(tf, 1), "flops": synth.gemm_flops(n, k, m),
                           "kernel": dec.last_kernel(),
                           "frac_measured_bf16": round(tf / peaks["bf16_tflops"], 4),
                           "frac_nominal_2250": round(tf / 2250.0, 4)}
                del xg, yg
            pre[f"M{m}"] = per
    top = pre["M4096"]
    tot_fl = sum(v["flops"] for v in top.values())
    tot_us = sum(v["us"] for v in top.values())
    roof = {"bound": "tensor", "workload": "prefill M=4096, the four 27B-class layer shapes, int4 sym g128",
            "per_shape": top, "layer_TFLOPs": round(tot_fl / tot_us / 1e6, 1),
            "achieved": round(tot_fl / tot_us / 1e6, 1), "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
            "frac": round(tot_fl / tot_us / 1e6 / peaks["bf16_tflops"], 4),
            "frac_of_nominal_2250": round(tot_fl / tot_us / 1e6 / 2250.0, 4)}
    return roof, pre


def tp_prefill(dec, dist, device, st, shapes, L, g):
    """One tensor-parallel prefill layer at M = 4096: column-parallel GEMMs need no exchange; a row-parallel GEMM runs
    in four token chunks and the NCCL f16 all-reduce of chunk i overlaps the GEMM of chunk i+1 (second stream)."""
    import torch
    m, chunks = 4096, 4
    cm = m // chunks
    comm = torch.cuda.Stream(device=device)
    xg = {nm: (torch.randn((m, shapes[nm][0]), generator=g, device=device, dtype=torch.float32)
               / (shapes[nm][0] ** 0.5)).to(torch.float16) for nm in LAYER_ORDER}
    yg = {nm: torch.empty((m, shapes[nm][1]), device=device, dtype=torch.float16) for nm in LAYER_ORDER}
    nl = min(L, 4)
    evs = [torch.cuda.Event() for _ in range(chunks)]

    def layers(overlap: bool):
        for li in range(nl):
            for nm in LAYER_ORDER:
                if shapes[nm][2] != "row":
                    dec.lin_forward(f"l{li}.{nm}", xg[nm], m, dst=yg[nm], out_f16=True)
                elif not overlap:
                    dec.lin_forward(f"l{li}.{nm}", xg[nm], m, dst=yg[nm], out_f16=True)
                    dist.all_reduce(yg[nm])
                else:
                    for c in range(chunks):
                        dec.lin_forward(f"l{li}.{nm}", xg[nm][c * cm:(c + 1) * cm], cm, dst=yg[nm][c * cm:(c + 1) * cm],
                                        out_f16=True)
                        evs[c].record(st)
                        comm.wait_event(evs[c])
                        with torch.cuda.stream(comm):
                            dist.all_reduce(yg[nm][c * cm:(c + 1) * cm])
                    st.wait_stream(comm)     # what follows a row-parallel layer consumes the summed output

    res = {}
    with torch.cuda.stream(st):
        for tag, ov in (("serial", False), ("overlapped", True)):
            layers(ov)
            st.synchronize()
            comm.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(st)
            for _ in range(2):
                layers(ov)
            e1.record(st)
            e1.synchronize()
            tms = torch.tensor([e0.elapsed_time(e1) / (2 * nl)], device=device)
            dist.all_reduce(tms, op=dist.ReduceOp.MAX)
            res[tag] = float(tms.item())
    fl = sum(synth.gemm_flops(synth.DENSE_27B[nm][1], synth.DENSE_27B[nm][0], m) for nm in LAYER_ORDER)
    # parity of the overlapped form: the summed o_proj output of the last layer against a plain torch reduction
    nm = "o_proj"
    ref = torch.empty_like(yg[nm])
    with torch.cuda.stream(st):
        dec.lin_forward(f"l{nl - 1}.{nm}", xg[nm], m, dst=ref, out_f16=True)
        st.synchronize()
    ref32 = ref.float()
    dist.all_reduce(ref32)
    err = float((yg[nm].float() - ref32).abs().max().item())
    best = min(res.values())
    return {"ms_per_layer": round(best, 4), "ms_per_layer_serial": round(res["serial"], 4),
            "ms_per_layer_overlapped": round(res["overlapped"], 4),
            "TFLOPs_all_gpus": round(fl / best / 1e9, 1),
            "allreduce": "NCCL f16 sum on o_proj and down outputs, four token chunks, overlapped with the next chunk's GEMM",
            "o_proj_f16_allreduce_vs_f32_sum_max_abs_err": err}


def moe_layer(dec, dist, device, st, rank, world, g):
    """One 35B-A3B-class MoE layer (128 experts, hidden 2048, expert FFN 768, top-8, g32) at T = 1, 64, 4096.
    N > 1: expert-parallel, 128/N experts per GPU; the timed call is moe_ffn plus the NCCL f16 all-reduce of the
    partial outputs, max over ranks; the result of T = 64 is compared with the CPU oracle on rank 0."""
    import torch
    mo = synth.MOE_35B
    ne, h, f, kk, grp = mo["n_experts"], mo["hidden"], mo["moe_ffn"], mo["top_k"], mo["group"]
    cnt = ne // world
    e0x = rank * cnt
    dec.set_moe(ne, kk, f, h, grp, expert_first=e0x, expert_count=cnt)
    nlay = 4   # rotate over 4 layers of experts (4 x 340 MB / N per GPU)
    full0 = None
    for li in range(nlay):
        # every rank generates the same full layer and keeps its own experts
        q13, s13 = synth.make_linear_cuda(ne * 2 * f, h, grp, seed=900 + li, device=device)
        q2, s2 = synth.make_linear_cuda(ne * h, f, grp, seed=950 + li, device=device)
        r13 = slice(e0x * 2 * f, (e0x + cnt) * 2 * f)
        r2 = slice(e0x * h, (e0x + cnt) * h)
        dec.upload_experts(li, q13[r13].contiguous(), s13[r13].contiguous(), q2[r2].contiguous(), s2[r2].contiguous())
        if li == 0 and rank == 0:
            full0 = tuple(a.cpu().numpy() for a in (q13, s13, q2, s2))
        del q13, s13, q2, s2
    res = {}
    with torch.cuda.stream(st):
        for T in (1, 64, 4096):
            lg = torch.randn((T, ne), generator=g, device=device, dtype=torch.float32)
            xm = torch.randn((T, h), generator=g, device=device, dtype=torch.float32).to(torch.float16)
            if world > 1:
                dist.broadcast(lg, 0)
                dist.broadcast(xm, 0)
            ym = torch.empty((T, h), device=device, dtype=torch.float16 if world > 1 else torch.float32)

            def call(li):
                dec.moe_ffn_dev_t(li, lg, xm, T, out=ym, out_f16=world > 1)
                if world > 1:
                    dist.all_reduce(ym)
            for li in range(nlay):
                call(li)
            st.synchronize()
            if world > 1:
                dist.barrier()
            # one GPU: the nlay calls replayed as a CUDA graph, the way the reference replays its decode chain;
            # expert-parallel: eager calls (the NCCL all-reduce of torch is not captured)
            gxm = None
            if world == 1:
                dec.capture_begin()
                for li in range(nlay):
                    call(li)
                gxm = dec.capture_end()
                dec.graph_launch(gxm)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 5
            e0.record(st)
            for _ in range(reps):
                if gxm is not None:
                    dec.graph_launch(gxm)
                else:
                    for li in range(nlay):
                        call(li)
            e1.record(st)
            e1.synchronize()
            if gxm is not None:
                dec.graph_destroy(gxm)
            us = e0.elapsed_time(e1) * 1e3 / (reps * nlay)
            if world > 1:
                tus = torch.tensor([us], device=device)
                dist.all_reduce(tus, op=dist.ReduceOp.MAX)
                us = float(tus.item())
            idx, _ = dec.moe_topk(lg)
            hit = int(torch.unique(idx).numel())
            wbytes = hit * (2 * f * h // 2 + 2 * f * (h // grp) * 2 + h * f // 2 + h * (f // grp) * 2)
            flops = 2 * T * kk * (h * 2 * f + f * h)
            res[f"T{T}"] = {"us": round(us, 1), "experts_hit": hit, "weight_GBps_all_gpus": round(wbytes / us / 1e3, 1),
                            "TFLOPs_all_gpus": round(flops / us / 1e6, 2)}
            if T == 64:
                call(0)
                st.synchronize()
                if rank == 0:
                    import oracle
                    oracle.build()
                    q13, s13, q2, s2 = full0
                    sub = np.arange(0, 64, 4)
                    want = oracle.moe_ffn(np.ascontiguousarray(xm.cpu().numpy().view(np.uint16)[sub]),
                                          np.ascontiguousarray(lg.cpu().numpy()[sub]),
                                          q13.view(np.uint32).reshape(ne, 2 * f, h // 8), s13.view(np.uint16).reshape(ne, 2 * f, h // grp),
                                          q2.view(np.uint32).reshape(ne, h, f // 8), s2.view(np.uint16).reshape(ne, h, f // grp), kk, grp)
                    err = float(np.abs(ym.float().cpu().numpy()[sub] - want).max())
                    res["T64"]["max_abs_err_vs_oracle_16_tokens"] = err
    if world > 1:
        res["expert_parallel"] = f"{cnt} experts per GPU, NCCL f16 all-reduce of the partial [T,{h}] outputs inside the timed call"
    return res


# ------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the per-shape / M sweep extras")
    ap.add_argument("--tune", action="append", default=[], help="library knob key=value (repeatable)")
    ap.add_argument("--case", default=None,
                    help="run ONE small case instead of the benchmark, for profilers: "
                         "gemv:<linear>:<m>, gemm:<linear>:<m> or moe:<tokens>, e.g. gemm:gate_up:4096 (prints its device time)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    run_b200_arm(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
