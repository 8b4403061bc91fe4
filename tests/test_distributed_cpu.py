"""The multi-rank host logic on CPU: two gloo ranks shard a workload, run the oracle on their
slices, and the slices reassemble to the unsharded result; timing aggregates as max over ranks."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import fused_attention_b200 as fa
from fused_attention_b200.workloads import Workload, workload_inputs
from oracle.naive_attention import attention as oracle


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


W = Workload("unit", B=2, R=4, L=96, H=16, sigma=1.0, seed=5)


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        shard = fa.shard_units(W.B, W.R, world, rank)
        q, k, v = workload_inputs(W, heads=slice(shard.h0, shard.h1), batches=slice(shard.b0, shard.b1))
        y = oracle(q, k, v, W.H)           # stands in for the GPU operator: same slicing, same layout
        my_flops = fa.attention_flops(shard.b1 - shard.b0, shard.h1 - shard.h0, W.L, W.H)
        my_seconds = 0.010 * (rank + 1)    # rank 1 is the slow one

        def red(op):
            def f(x):
                t = torch.tensor([x], dtype=torch.float64)
                dist.all_reduce(t, op=op)
                return float(t.item())
            return f

        agg = fa.aggregate_throughput(my_flops, my_seconds, red(dist.ReduceOp.SUM), red(dist.ReduceOp.MAX))
        torch.save({"shard": shard, "y": y, "agg": agg}, os.path.join(out_dir, f"rank{rank}.pt"))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_ranks_shard_and_aggregate(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    q, k, v = workload_inputs(W)
    full = oracle(q, k, v, W.H)
    rebuilt = torch.zeros_like(full)
    for rank in range(world):
        d = torch.load(os.path.join(tmp_path, f"rank{rank}.pt"), weights_only=False)
        s = d["shard"]
        rebuilt[s.b0:s.b1, :, s.h0 * W.H:s.h1 * W.H] = d["y"]
        assert d["agg"]["total_flops"] == fa.attention_flops(W.B, W.R, W.L, W.H)
        assert abs(d["agg"]["seconds"] - 0.020) < 1e-12          # max over ranks, not the sum or mean
        assert abs(d["agg"]["tflops"] - d["agg"]["total_flops"] / 0.020 / 1e12) < 1e-9
    assert float((rebuilt - full).abs().max()) <= 1e-6
