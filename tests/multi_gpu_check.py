"""Parity of the tensor-/expert-parallel path on N GPUs of one node.  Not collected by pytest; run with
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29511 tests/multi_gpu_check.py
Every rank uploads its shard (llm170_b200/shard.py), runs the CUDA kernels through the C ABI, the partial
results are combined with NCCL exactly as bench.py does, and rank 0 compares with the CPU oracle."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from llm170_b200 import shard, synth  # noqa: E402
from llm170_b200.w4a16_dec import W4a16Dec  # noqa: E402


def main():
    rank, world, lr = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    dist.init_process_group("nccl", device_id=dev)
    dec = W4a16Dec(lr)
    n, k, g = 1024, 2048, 128
    q, s = synth.make_linear(n, k, g, seed=9)
    worst = 0.0
    for t in (1, 8, 64):
        x = synth.make_acts(t, k, seed=t, scale=1.0 if t <= 8 else 1 / np.sqrt(k))
        want = oracle.linear_lane(q, s, x, t, n, k, g) if rank == 0 else None
        # column-parallel: all-gather of the row slices
        qs, ss, n_s, k_s = shard.shard_linear(q, s, n, k, g, "col", rank, world)
        dec.upload_lin_g("col", qs, ss, n_s, k_s, g)
        y = dec.lin_forward("col", torch.from_numpy(x.view(np.float16).copy()).to(dev), t)
        parts = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(parts, y)
        col = torch.cat(parts, dim=1).cpu().numpy()
        # row-parallel: f16 partial outputs, NCCL all-reduce
        qs, ss, n_s, k_s = shard.shard_linear(q, s, n, k, g, "row", rank, world)
        dec.upload_lin_g("row", qs, ss, n_s, k_s, g)
        xs = shard.shard_acts(x, k, "row", rank, world)
        yr = dec.lin_forward("row", torch.from_numpy(xs.view(np.float16).copy()).to(dev), t, out_f16=True)
        dist.all_reduce(yr)
        if rank == 0:
            e_col = float(np.abs(col - want).max())
            e_row = float(np.abs(yr.float().cpu().numpy() - want).max())
            scale = float(np.abs(want).max())
            print(f"t={t}: column-parallel max err {e_col:.2e}, row-parallel(f16 all-reduce) max err {e_row:.2e} (|y|max {scale:.2f})")
            worst = max(worst, e_col, e_row / max(1.0, scale))
            assert e_col <= 2e-3 and e_row <= 2e-3 * max(1.0, scale) * 2
    # row-parallel with the all-reduce fused into the GEMV kernel (peer stores), eager and graph-replayed; the last shape
    # leaves every rank a K slice of six scale groups, fewer than the row-block form's eight warps
    dec.tp_setup(rank, world, max_rows=2048)
    shapes = [(1024, 2048, 128), (512, 4096, 128), (2048, 1024, 32), (768, 768 * world, 128)]
    lins = []
    for i, (n2, k2, g2) in enumerate(shapes):
        q2, s2 = synth.make_linear(n2, k2, g2, seed=20 + i)
        qs, ss, n_s, k_s = shard.shard_linear(q2, s2, n2, k2, g2, "row", rank, world)
        dec.upload_lin_g(f"ar{i}", qs, ss, n_s, k_s, g2)
        lins.append((q2, s2, n2, k2, g2))
    for t in (1, 8):
        for rep in range(3):
            for i, (q2, s2, n2, k2, g2) in enumerate(lins):
                x = synth.make_acts(t, k2, seed=100 * rep + i + t)
                xs = torch.from_numpy(shard.shard_acts(x, k2, "row", rank, world).view(np.float16).copy()).to(dev)
                y = dec.sk_single_allreduce(f"ar{i}", xs, t=t)
                dec.kernel_status()
                if rank == 0:
                    err = float(np.abs(y.cpu().numpy() - oracle.linear_lane(q2, s2, x, t, n2, k2, g2)).max())
                    worst = max(worst, err)
                    assert err <= 2e-3, (t, rep, i, err)
    st = torch.cuda.ExternalStream(dec.stream_ptr(), device=dev)
    # A long replay: the same 4-launch graph (all three row-parallel linears, one of them twice) 2000 times with
    # the inputs rewritten between replays (8 rotating input sets); every 100th replay is compared with the oracle.
    # Every wait is bounded, so a lost word would end as a status code, not as a hang.
    nsets = 8
    xsets, wants = [], []
    for si in range(nsets):
        row = []
        for i, (q2, s2, n2, k2, g2) in enumerate(lins):
            x = synth.make_acts(1, k2, seed=5000 + 10 * si + i)
            row.append(torch.from_numpy(shard.shard_acts(x, k2, "row", rank, world).view(np.float16).copy()).to(dev))
            if rank == 0:
                wants.append(oracle.linear_lane(q2, s2, x, 1, n2, k2, g2))
        xsets.append(row)
    xin = [torch.empty_like(t) for t in xsets[0]]
    outs = [torch.zeros((1, lins[i][2]), device=dev) for i in (0, 1, 2, 0)]
    torch.cuda.synchronize()
    dist.barrier()
    with torch.cuda.stream(st):
        for j, i in enumerate((0, 1, 2, 0)):
            dec.sk_single_allreduce(f"ar{i}", xin[i], out=outs[j], t=1)       # warm
        st.synchronize()
        dist.barrier()
        dec.capture_begin()
        for j, i in enumerate((0, 1, 2, 0)):
            dec.sk_single_allreduce(f"ar{i}", xin[i], out=outs[j], t=1)
        gx = dec.capture_end()
        replays, checked = 2000, 0
        for rep in range(replays):
            si = rep % nsets
            for i in range(3):
                xin[i].copy_(xsets[si][i], non_blocking=True)
            dec.graph_launch(gx)
            if rep % 100 == 99 or rep == replays - 1:
                dec.sync()
                if rank == 0:
                    for j, i in enumerate((0, 1, 2, 0)):
                        err = float(np.abs(outs[j].cpu().numpy() - wants[si * len(lins) + i]).max())
                        worst = max(worst, err)
                        assert err <= 2e-3, (rep, j, err)
                checked += 1
        dec.sync()
        dec.graph_destroy(gx)
    if rank == 0:
        print(f"fused all-reduce GEMV over {world} ranks (eager + {replays} graph replays, {checked} checked): worst max err {worst:.2e}")
    dist.barrier()
    # A wait that runs out: with the limit shortened to 2^20 cycles (half a millisecond), rank 0 makes one fused
    # launch that no peer joins.  Its wait gives up and the status call reports it; the kernel returns, the context
    # stays usable.  Then every rank re-arms between two barriers and the next launches are correct again.
    dec.set_tuning("tp_wait_log2", 20)
    q2, s2, n2, k2, g2 = lins[0]
    x = synth.make_acts(1, k2, seed=777)
    xs = torch.from_numpy(shard.shard_acts(x, k2, "row", rank, world).view(np.float16).copy()).to(dev)
    if rank == 0:
        dec.sk_single_allreduce("ar0", xs, t=1)
        gave_up = False
        try:
            dec.sync()
        except Exception as e:   # W4a16Error: a bounded pipeline wait expired
            gave_up = "wait expired" in str(e)
        assert gave_up, "the lone launch should have reported an expired wait"
    dist.barrier()
    dec.tp_rearm()
    dist.barrier()
    dec.set_tuning("tp_wait_log2", 31)
    for rep in range(3):
        y = dec.sk_single_allreduce("ar0", xs, t=1)
        dec.sync()
        if rank == 0:
            err = float(np.abs(y.cpu().numpy() - oracle.linear_lane(q2, s2, x, 1, n2, k2, g2)).max())
            assert err <= 2e-3, ("after re-arm", rep, err)
    if rank == 0:
        print("expired wait reported, collective re-arm, next launches correct")
    dist.barrier()
    # expert-parallel MoE
    ne, kk, f, h, t = 16, 4, 128, 256, 40
    w = synth.make_experts(ne, f, h, 32, seed=3)
    xm = synth.make_acts(t, h, seed=4)
    lg = synth.make_router_logits(t, ne, seed=5)
    e0, cnt = shard.expert_range(ne, rank, world)
    dec.set_moe(ne, kk, f, h, 32, expert_first=e0, expert_count=cnt)
    dec.upload_experts(0, *[a[e0:e0 + cnt] for a in w])
    y = dec.moe_ffn_dev_t(0, torch.from_numpy(lg).to(dev), torch.from_numpy(xm.view(np.float16).copy()).to(dev), t)
    dist.all_reduce(y)
    dec.sync()
    if rank == 0:
        err = float(np.abs(y.cpu().numpy() - oracle.moe_ffn(xm, lg, *w, kk, 32)).max())
        print(f"expert-parallel MoE over {world} ranks: max err {err:.2e}")
        assert err <= 2e-3
        print("MULTI_GPU_CHECK OK")
    dist.barrier()
    dist.destroy_process_group()
    dec.close()


if __name__ == "__main__":
    main()
