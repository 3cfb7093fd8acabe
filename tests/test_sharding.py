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


# ---- packed rows: whole documents, token-balanced -------------------------------------------------------------------

def test_document_ranges_cover_balance_and_rebase():
    sys.path.insert(0, ROOT)
    from cute_triadic_gdn_b200.sharding import document_ranges, head_slice, shard_documents
    from oracle import triadic_oracle as orc
    cu = orc.lognormal_documents(131072, seed=11)
    n_docs, total = cu.numel() - 1, int(cu[-1])
    for parts in (1, 2, 4, 8):
        rs = document_ranges(cu, parts)
        assert len(rs) == parts and rs[0].doc_lo == 0 and rs[-1].doc_hi == n_docs
        assert all(a.doc_hi == b.doc_lo and a.tok_hi == b.tok_lo for a, b in zip(rs, rs[1:]))     # contiguous cover
        longest = int((cu[1:] - cu[:-1]).max())
        assert max(r.tok_hi - r.tok_lo for r in rs) <= total / parts + longest                    # as even as documents allow
    # fewer documents than parts: some parts are empty, nothing is lost
    rs = document_ranges([0, 100, 164], 4)
    assert sum(r.doc_hi - r.doc_lo for r in rs) == 2 and rs[-1].tok_hi == 164
    x = torch.arange(164.).view(1, 164, 1)
    views, sub, rng = shard_documents([x], torch.tensor([0, 100, 164], dtype=torch.int32), 2, 1)
    assert sub.tolist() == [0, 64] and views[0].is_contiguous() and views[0][0, 0, 0] == 100 and rng.tok_lo == 100
    assert head_slice(32, 8, 3) == slice(12, 16)
    with pytest.raises(ValueError):
        head_slice(30, 8, 0)
    with pytest.raises(ValueError):
        document_ranges([0, 5, 5], 2)


def _packed_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    from cute_triadic_gdn_b200.sharding import shard_documents
    from oracle import triadic_oracle as orc
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    T, H, E = 320, 2, 2
    cu = torch.tensor([0, 64, 65, 200, 320], dtype=torch.int32)
    ins = orc.make_inputs(1, T, H, E, seed=5)
    do = orc.make_grad_output((1, T, H, 128), 6)
    views, sub, rng = shard_documents(list(ins) + [do], cu, world, rank)
    mine = [t.contiguous() for t in views[:7]]
    o, grads = orc.reference_with_grads(orc.chunk_reference, mine, views[7].contiguous(), cu_seqlens=sub, dtype=torch.float32)
    tokens = torch.tensor([float(rng.tok_hi - rng.tok_lo)])
    dist.all_reduce(tokens)                                # the ranks' token counts add up to the whole row
    assert tokens.item() == float(T)
    torch.save({"o": o, "grads": grads}, os.path.join(out_dir, f"packed{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_documents_shard_without_exchange(tmp_path):
    """Two ranks take token-balanced ranges of whole documents; their results, concatenated along the token axis, are the
    single-process result: a document never needs anything from another one."""
    sys.path.insert(0, ROOT)
    from oracle import triadic_oracle as orc
    world = 2
    mp.spawn(_packed_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    parts = [torch.load(os.path.join(tmp_path, f"packed{r}.pt")) for r in range(world)]
    cu = torch.tensor([0, 64, 65, 200, 320], dtype=torch.int32)
    ins = orc.make_inputs(1, 320, 2, 2, seed=5)
    do = orc.make_grad_output((1, 320, 2, 128), 6)
    o, grads = orc.reference_with_grads(orc.chunk_reference, ins, do, cu_seqlens=cu, dtype=torch.float32)
    assert torch.allclose(torch.cat([p["o"] for p in parts], 1), o, atol=1e-6)
    for i in range(7):
        assert torch.allclose(torch.cat([p["grads"][i] for p in parts], 1), grads[i], atol=1e-5)
