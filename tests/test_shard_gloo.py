"""The N>1 partitioning, exercised by two real ranks on CPU (gloo): every rank computes its shard with the
CPU oracle and the ranks' results are combined with the collective the GPU path uses (none for
column-parallel, all-reduce sum for row-parallel and for expert-parallel MoE)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    from llm170_b200 import shard, synth
    n, k, group, t = 256, 512, 128, 3
    q, s = synth.make_linear(n, k, group, seed=1)
    x = synth.make_acts(t, k, seed=2)
    full = oracle.linear_lane(q, s, x, t, n, k, group, nthreads=2)
    # column-parallel with a fused gate|up split per half: concatenate, no reduction
    qs, ss, n_s, k_s = shard.shard_linear(q, s, n, k, group, "col", rank, world, fused_halves=2)
    y = torch.from_numpy(oracle.linear_lane(qs, ss, shard.shard_acts(x, k, "col", rank, world), t, n_s, k_s, group, nthreads=2))
    parts = [torch.empty_like(y) for _ in range(world)]
    dist.all_gather(parts, y)
    half = n_s // 2
    col = np.concatenate([p[:, :half].numpy() for p in parts] + [p[:, half:].numpy() for p in parts], axis=1)
    ok_col = np.array_equal(col, full)
    # row-parallel: partial sums all-reduced
    qs, ss, n_s, k_s = shard.shard_linear(q, s, n, k, group, "row", rank, world)
    y = torch.from_numpy(oracle.linear_lane(qs, ss, shard.shard_acts(x, k, "row", rank, world), t, n_s, k_s, group, nthreads=2))
    dist.all_reduce(y)
    ok_row = float(np.abs(y.numpy() - full).max()) < 1e-4
    # expert-parallel MoE: local partial FFN outputs all-reduced
    ne, kk, f, h = 8, 2, 64, 128
    w = synth.make_experts(ne, f, h, 32, seed=3)
    xm = synth.make_acts(5, h, seed=4)
    lg = synth.make_router_logits(5, ne, seed=5)
    e0, cnt = shard.expert_range(ne, rank, world)
    part = torch.from_numpy(oracle.moe_ffn(xm, lg, *w, kk, 32, experts=(e0, e0 + cnt)))
    dist.all_reduce(part)
    ok_moe = float(np.abs(part.numpy() - oracle.moe_ffn(xm, lg, *w, kk, 32)).max()) < 1e-6
    if rank == 0:
        open(os.path.join(out_dir, "result"), "w").write(f"{ok_col} {ok_row} {ok_moe}")
    dist.destroy_process_group()


def test_two_rank_sharding_on_cpu(tmp_path):
    import oracle
    oracle.build()
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert open(tmp_path / "result").read() == "True True True"


def test_shard_contracts():
    from llm170_b200 import shard, synth
    q, s = synth.make_linear(64, 256, 128, seed=0)
    with pytest.raises(ValueError):
        shard.shard_linear(q, s, 64, 256, 128, "row", 0, 4)       # 64-channel slices would split a scale group
    with pytest.raises(ValueError):
        shard.shard_linear(q, s, 64, 256, 128, "col", 0, 8)       # fewer than 16 rows per rank
    with pytest.raises(ValueError):
        shard.expert_range(6, 0, 4)
    qs, ss, n_s, k_s = shard.shard_linear(q, s, 64, 256, 128, "row", 1, 2)
    assert (n_s, k_s) == (64, 128) and qs.shape == (64, 16) and ss.shape == (64, 1)
    assert shard.expert_range(128, 3, 8) == (48, 16)
