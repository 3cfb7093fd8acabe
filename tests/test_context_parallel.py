"""Context-parallel schedule on the CPU: three gloo ranks hold consecutive token slices of the same sequences, the per-segment
operator is a differentiable torch statement of the token-by-token recurrence (cute_triadic_gdn/ops/gdn_joint.py:1-8) with
the state handed in and out, and `context_parallel_joint` moves the states forward and their gradients backward between
the ranks, two head groups in flight.  Outputs and all seven gradients must equal those of the unsplit sequences."""
import os
import socket
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def segment_reference(q, k, v, k2, q2, g, beta, state_in, scale):
    """Token by token in f64, differentiable through state_in and state_out: (o, state_out)."""
    B, T, H, D = q.shape
    E = k2.shape[-1]
    S = torch.zeros(B, H, E, D, D, dtype=torch.float64) if state_in is None else state_in
    rows = []
    for t in range(T):
        S = S * g[:, t].exp()[..., None, None]
        kap = k2[:, t, :, :, None] * k[:, t, :, None, :]
        pred = torch.einsum('bhed,bhedv->bhv', kap, S)
        S = S + beta[:, t, :, None, None, None] * kap[..., None] * (v[:, t] - pred)[:, :, None, None, :]
        qk = q2[:, t, :, :, None] * q[:, t, :, None, :]
        rows.append(torch.einsum('bhed,bhedv->bhv', qk, S) * scale)
    return torch.stack(rows, 1), S


def make(B, T, H, E, D, seed):
    gen = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=gen, dtype=torch.float64)
    l2 = lambda t: t / t.norm(dim=-1, keepdim=True)
    ins = [l2(r(B, T, H, D)), l2(r(B, T, H, D)), r(B, T, H, D), l2(r(B, T, H, E).abs()), l2(r(B, T, H, E).abs()),
           -torch.nn.functional.softplus(r(B, T, H, E)) * 0.3, torch.sigmoid(r(B, T, H))]
    return ins, r(B, T, H, D)


SHAPE = (2, 24, 4, 2, 8)          # B, T, H, E, D: a tiny head dimension keeps the f64 loop fast


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    from cute_triadic_gdn_b200.context_parallel import context_parallel_joint
    B, T, H, E, D = SHAPE
    ins, do = make(B, T, H, E, D, 5)
    tl = T // world
    sl = slice(rank * tl, (rank + 1) * tl)
    mine = [t[:, sl].clone().requires_grad_(True) for t in ins]
    o = context_parallel_joint(*mine, head_groups=2, scale=D ** -0.5, segment_fn=segment_reference,
                               state_dtype=torch.float64)
    (o * do[:, sl]).sum().backward()
    torch.save({"o": o.detach(), "grads": [t.grad for t in mine]}, os.path.join(out_dir, f"rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_three_ranks_match_the_unsplit_sequences(tmp_path):
    world = 3
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    parts = [torch.load(os.path.join(tmp_path, f"rank{r}.pt")) for r in range(world)]
    B, T, H, E, D = SHAPE
    ins, do = make(B, T, H, E, D, 5)
    leaves = [t.clone().requires_grad_(True) for t in ins]
    o, _ = segment_reference(*leaves, None, D ** -0.5)
    (o * do).sum().backward()
    assert torch.allclose(torch.cat([p["o"] for p in parts], 1), o.detach(), rtol=1e-10, atol=1e-12)
    for i, leaf in enumerate(leaves):
        got = torch.cat([p["grads"][i] for p in parts], 1)
        assert torch.allclose(got, leaf.grad, rtol=1e-9, atol=1e-11), i


def test_head_groups():
    sys.path.insert(0, ROOT)
    from cute_triadic_gdn_b200.context_parallel import head_groups_of
    assert head_groups_of(8, 2) == [(0, 4), (4, 8)]
    assert head_groups_of(3, 8) == [(0, 1), (1, 2), (2, 3)]
    assert head_groups_of(5, 2) == [(0, 2), (2, 5)]
    assert head_groups_of(4, 1) == [(0, 4)]
