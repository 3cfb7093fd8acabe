"""Multi-GPU plan of the benchmark, exercised with two gloo ranks on the CPU: every rank takes its own contiguous slice of
heads, computes independently (here: the CPU oracle on a tiny problem), and only the timing is reduced over ranks.
Also checks that concatenating the per-rank results along the head axis reproduces the single-process result, i.e. that
the path really shards with no exchange step."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    from oracle import triadic_oracle as orc
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    B, T, H, E = 1, 128, 4, 2
    ins = orc.make_inputs(B, T, H, E, seed=3)
    do = orc.make_grad_output((B, T, H, 128), 4)
    hl = H // world
    sl = slice(rank * hl, (rank + 1) * hl)
    mine = [t[:, :, sl].contiguous() for t in ins]
    dist.barrier()
    o, grads = orc.reference_with_grads(orc.chunk_reference, mine, do[:, :, sl].contiguous(), dtype=torch.float32)
    ms = torch.tensor([float(rank + 1)])               # stands in for the per-rank elapsed time
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    assert ms.item() == float(world)
    torch.save({"o": o, "grads": grads}, os.path.join(out_dir, f"rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_heads_shard_without_exchange(tmp_path):
    sys.path.insert(0, ROOT)
    from oracle import triadic_oracle as orc
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    parts = [torch.load(os.path.join(tmp_path, f"rank{r}.pt")) for r in range(world)]
    ins = orc.make_inputs(1, 128, 4, 2, seed=3)
    do = orc.make_grad_output((1, 128, 4, 128), 4)
    o, grads = orc.reference_with_grads(orc.chunk_reference, ins, do, dtype=torch.float32)
    assert torch.allclose(torch.cat([p["o"] for p in parts], 2), o, atol=1e-6)
    for i in range(7):
        assert torch.allclose(torch.cat([p["grads"][i] for p in parts], 2), grads[i], atol=1e-5)


def test_bench_reference_arm_runs_only_on_rank_zero(monkeypatch, capsys):
    sys.path.insert(0, ROOT)
    import bench

    class Args:
        workload, steps, warmup, gpus = "small", 1, 0, 2

    bench.run_reference(Args, rank=1, world=2)
    assert capsys.readouterr().out == ""
