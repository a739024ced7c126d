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
